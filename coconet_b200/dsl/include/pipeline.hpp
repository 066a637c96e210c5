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
  // Non-aborting form of the same check.
  bool canFuse(const std::vector<NodeRef> &stages, std::string *why = nullptr) const;

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
};

}  // namespace ACCCDSL
