// Pipeline: the stages reachable from a set of outputs, fusion groups over
// them, and code generation.  Surface of the reference's src/pipeline.hpp:
// 499-684 as far as the data-parallel example programs use it.
#pragma once

#include <iostream>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "dsl.hpp"

namespace ACCCDSL {

// Which optimizer a fused ReduceScatter -> update -> AllGather group computes,
// with the DSL objects playing each role (empty name = absent, value 1).
struct FusedUpdate {
  enum Rule { Unknown = 0, SGD, Adam, LAMB } rule = Unknown;
  NodeRef grad, weight, m, v;                 // tensors
  std::string lr, beta1, beta2, decay;        // Variable names
  // Mixed precision: `weight` is the fp32 master (a Sliced tensor: every rank
  // keeps its own slice) and `lp` the 16-bit Replicated copy that is gathered
  // to all ranks (the halfw argument of the reference's hook,
  // src/codegen.cpp:1910).  Absent otherwise.
  NodeRef lp;
  // The reduced gradient is multiplied (or, with gscale_div, divided) by this
  // Variable before it is used: the loss scale of mixed-precision training.
  std::string gscale;
  bool gscale_div = false;
};

// Schedule transformations (surface of the reference's src/pipeline.hpp:51-54,
// 76-79, 552-558).
enum SplitType { AllReduceRSAG, AllReduceBR };
struct ReorderedStages {
  std::vector<Stage> compStages;       // the computations, now on slices
  std::vector<Stage> allGatherStages;  // one AllGather per Replicated tensor they update
};

class Pipeline {
 public:
  Pipeline(const std::string &name, std::initializer_list<Expression> args,
           std::initializer_list<Stage> outputs);

  const std::string &name() const { return name_; }

  // Fuse stages into one group (one kernel, or one fused collective when the
  // group contains ReduceScatter/AllGather).  Aborts with a message if the
  // stages are not part of the pipeline or the fusion would create a cycle.
  void fuse(std::initializer_list<Stage> stages);
  void fuse(const std::vector<Stage> &stages);
  // Non-aborting form of the same check.
  bool canFuse(const std::vector<NodeRef> &stages, std::string *why = nullptr) const;
  // Dissolve every fusion group (each stage on its own again).
  void unfuse() { fused_.clear(); }

  // ---- schedule transformations: AR_C -> RS_C_AG -> fused, without rewriting the program ----
  // split(AllReduceRSAG): the AllReduce stage becomes ReduceScatter + AllGather.
  // Returns {reduce-scatter stage, all-gather stage}; the all-gather stage IS
  // the handle that was passed in (stages that used it keep working).
  std::pair<Stage, Stage> split(Stage allReduce, SplitType type);
  // reorder: move `allGather` below the pointwise stages `comps` that consume
  // it, so that they compute on the rank's slice only; every Replicated tensor
  // they update gets an AllGather of its own.
  ReorderedStages reorder(std::vector<Stage> comps, Stage allGather);
  // asSlice: keep a Replicated tensor (optimizer state) as a Sliced one; the
  // AllGather that fed its Update disappears.
  void asSlice(Tensor replicated);
  void asSlice(std::vector<Tensor> replicated);

  // Emit the CUDA host program.
  void codegen(const std::string &filename);
  void codegen(std::ostream &os);

  void print(std::ostream &os) const;

  // Introspection used by the emitter and by tests.
  const std::vector<NodeRef> &stages() const { return stages_; }                 // topological
  std::vector<std::vector<NodeRef>> groups() const;                               // topological
  // Recognise the update rule of a fused group by evaluating the DAG on
  // sample values against the closed forms (role assignment by search).
  FusedUpdate classify(const std::vector<NodeRef> &group) const;

 private:
  std::string name_;
  std::vector<NodeRef> args_;
  std::vector<NodeRef> outputs_;
  std::vector<NodeRef> stages_;
  std::vector<std::set<const Node *>> fused_;
  void rediscover();  // recompute stages_ after a transformation
};

// Derives the schedules of the CoCoNet paper from ONE pipeline written as
// AllReduce + computation, and emits a program for each (surface of the
// reference's src/pipeline.hpp:675-684; there it enumerates and prints):
//   <dir>/<name>-AR_C.cu          as written, computations fused into kernels
//   <dir>/<name>-RS_C_AG.cu       split + reorder + asSlice(canSlice)
//   <dir>/<name>-fuse_RS_C_AG.cu  everything fused into one kernel
// The programs are timed by building and running them (python -m
// coconet_b200.dsl.autotune --derive ...): measuring needs the GPUs, emitting
// does not.  The pipeline is left in its last (fused) schedule.
class Autotuner {
 public:
  Autotuner() {}
  void setOutputDir(const std::string &dir) { dir_ = dir; }
  void autotune(Pipeline &pipeline) { autotune(pipeline, std::vector<Tensor>()); }
  // canSlice: Replicated tensors that only the update itself reads and writes
  // (optimizer state): they become Sliced in the last two schedules.
  void autotune(Pipeline &pipeline, std::vector<Tensor> canSlice);
  const std::vector<std::string> &emitted() const { return emitted_; }  // files written

 private:
  std::string dir_ = ".";
  std::vector<std::string> emitted_;
};

}  // namespace ACCCDSL
