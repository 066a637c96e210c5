// Emitter: Pipeline -> one CUDA host program.
//
// Fused ReduceScatter -> update -> AllGather groups become ONE call into the
// C-ABI runtime (include/coconet_rt.h), chosen by Pipeline::classify from what
// the group computes -- where the reference returns a hard-coded
// AllReduce_pipe(...) string keyed on the pipeline's name and patches NCCL
// sources (src/codegen.cpp:1906-1947).  Stand-alone collectives become stock
// NCCL calls and pointwise groups generated kernels, the shape of the
// reference's unfused schedules (src/codegen.cpp:4146-4189, 1245-1285).  The
// emitted main() keeps the reference's structure and its
// "{SZ: .., Epochs: .., <stage>: .., Total: ..}" report line
// (src/codegen.cpp:4583-4784) but starts without MPI.
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <map>
#include <set>
#include <sstream>

#include "pipeline.hpp"

namespace ACCCDSL {

void ownedNodes(const NodeRef &n, bool root, std::vector<NodeRef> *out);

namespace {

[[noreturn]] void fail(const std::string &msg) {
  std::fprintf(stderr, "coconet codegen: %s\n", msg.c_str());
  std::exit(2);
}

const char *cocoType(TensorElemType t) {
  switch (t) {
    case Float32: return "cocoFloat32";
    case Float16: return "cocoFloat16";
    default: fail("the fused step supports Float32 and Float16 gradients only");
  }
}
const char *ncclType(TensorElemType t) {
  switch (t) {
    case Float32: return "ncclFloat32";
    case Float16: return "ncclFloat16";
    case Float64: return "ncclFloat64";
    case Int32: return "ncclInt32";
    default: fail("no NCCL type for this element type");
  }
}

std::string fmtConst(double v, TensorElemType t) {
  std::ostringstream o;
  o.precision(17);
  o << v;
  std::string s = o.str();
  if (t == Float32 || t == Float16) {
    if (s.find('.') == std::string::npos && s.find('e') == std::string::npos) s += ".0";
    s += "f";
  }
  return s;
}

// One launch of the emitted step function.
struct Step {
  enum Kind { Fused, FusedGeneric, Collective, Kernel, NormReduce } kind;
  std::string label;                 // timer name
  std::vector<NodeRef> stages;       // Kernel: stages computed; else one stage
  FusedUpdate fused;
  NodeRef coll;                      // Collective: the collective node
  int kernel_id = -1;
  // FusedGeneric: the gradient, the gathered weight tensor and the value gathered into it
  NodeRef ggrad, gweight, gvalue, greduce;
};

struct Emitter {
  const Pipeline &p;
  std::vector<NodeRef> args;
  NodeRef size_var;                               // the tensors' element count Variable
  std::vector<Step> steps;
  std::set<const Node *> in_memory;               // stage values that live in a buffer
  std::map<const Node *, std::string> buffer;     // stage -> buffer name
  bool needs_nccl = false;
  std::ostringstream kernels;

  explicit Emitter(const Pipeline &pp, const std::vector<NodeRef> &a) : p(pp), args(a) {
    for (const NodeRef &n : args)
      if (n->kind == NodeKind::Tensor) {
        if (!size_var) size_var = n->dim;
        else if (size_var.get() != n->dim.get())
          fail("all tensors of a pipeline must share one size Variable");
      }
    if (!size_var) fail("pipeline without tensors");
  }

  std::string N() const { return size_var->name; }
  std::string sliceCount() const { return "DIVUP(" + N() + ", comm_size)"; }

  // Where a stage's value can be read from memory: the tensor an Update wrote,
  // the gradient buffer a collective reduced in place, or an intermediate.
  bool collectiveRoot(const NodeRef &s, NodeRef *coll) const {
    NodeRef n = s;
    if (n->kind == NodeKind::Update) n = n->in[1];
    if (isCollective(n->kind)) {
      *coll = n;
      return true;
    }
    return false;
  }

  // ---- planning -------------------------------------------------------------
  void plan() {
    int kernel_id = 0;
    for (const auto &group : p.groups()) {
      bool has_coll = false, has_point = false;
      for (const NodeRef &s : group) {
        std::vector<NodeRef> own;
        ownedNodes(s, true, &own);
        for (const NodeRef &n : own) {
          if (isCollective(n->kind)) has_coll = true;
          else if (n->kind == NodeKind::Binary || n->kind == NodeKind::Sqrt || n->kind == NodeKind::Norm)
            has_point = true;
        }
      }
      if (has_coll && (has_point || group.size() > 1)) {
        Step st;
        st.kind = Step::Fused;
        st.stages = group;
        st.fused = p.classify(group);
        st.label = "FusedAllReduce";
        if (st.fused.rule == FusedUpdate::Unknown) {
          // not one of the rules the library ships a kernel for: compile the
          // group's arithmetic into a device functor for the generic fused kernel
          std::string why;
          if (!genericFusable(group, &st, &why)) {
            std::string names;
            for (const NodeRef &s : group) names += " " + s->name;
            fail("fused group {" + names + " } of pipeline '" + p.name() +
                 "' is not a ReduceScatter -> SGD | Adam | LAMB update -> AllGather step, and cannot "
                 "be compiled into a generic fused step either: " + why);
          }
          st.kind = Step::FusedGeneric;
          st.kernel_id = kernel_id++;
        }
        steps.push_back(st);
        continue;
      }
      if (has_coll) {  // a single collective stage
        NodeRef coll;
        if (!collectiveRoot(group[0], &coll)) fail("collective nested inside arithmetic in " + group[0]->name);
        Step st;
        st.kind = Step::Collective;
        st.stages = group;
        st.coll = coll;
        st.label = coll->kind == NodeKind::AllReduce ? "AllReduce"
                   : coll->kind == NodeKind::ReduceScatter ? "ReduceScatter"
                   : coll->kind == NodeKind::AllGather ? "AllGather" : "Broadcast";
        // fp32 sums run on the runtime's own collectives; anything else on stock NCCL
        if (!(coll->type == Float32 && coll->kind != NodeKind::Broadcast &&
              (coll->kind == NodeKind::AllGather || coll->red == Summation)))
          needs_nccl = true;
        steps.push_back(st);
        continue;
      }
      // pointwise group: cut at Norm stages (each is a reduction of its own)
      std::vector<NodeRef> segment;
      auto flush = [&]() {
        if (segment.empty()) return;
        Step st;
        st.kind = Step::Kernel;
        st.stages = segment;
        st.kernel_id = kernel_id++;
        st.label = "binOpFunc" + std::to_string(st.kernel_id);
        steps.push_back(st);
        segment.clear();
      };
      for (const NodeRef &s : group) {
        if (s->kind == NodeKind::Norm) {
          flush();
          Step st;
          st.kind = Step::NormReduce;
          st.stages = {s};
          st.label = "Norm" + s->name;
          steps.push_back(st);
        } else {
          segment.push_back(s);
        }
      }
      flush();
    }
    // A stage value read by a later step must be in memory.
    std::map<const Node *, int> computed_in;
    for (size_t k = 0; k < steps.size(); ++k)
      for (const NodeRef &s : steps[k].stages) computed_in[s.get()] = (int)k;
    for (size_t k = 0; k < steps.size(); ++k)
      for (const NodeRef &s : steps[k].stages) {
        std::vector<NodeRef> own;
        ownedNodes(s, true, &own);
        for (const NodeRef &n : own)
          for (const NodeRef &c : n->in)
            if (c->stage_id >= 0 && computed_in.count(c.get()) && computed_in[c.get()] != (int)k)
              in_memory.insert(c.get());
      }
    for (const NodeRef &s : p.stages())
      if (in_memory.count(s.get()) && s->kind != NodeKind::Update && !isCollective(s->kind))
        buffer[s.get()] = s->name;
  }

  // ---- generic fused groups ------------------------------------------------------
  // ReduceScatter(sum) of one Local tensor, any pointwise arithmetic (no Norm),
  // Updates of Sliced tensors, and exactly one Replicated tensor updated with
  // an AllGather of a Sliced value.
  bool genericFusable(const std::vector<NodeRef> &group, Step *st, std::string *why) const {
    std::vector<NodeRef> nodes;
    for (const NodeRef &s : group) ownedNodes(s, true, &nodes);
    for (const NodeRef &n : nodes) {
      if (n->kind == NodeKind::Norm) return *why = "it contains a Norm", false;
      if (n->kind == NodeKind::AllReduce || n->kind == NodeKind::Broadcast)
        return *why = "only ReduceScatter ... AllGather groups fuse", false;
      if (n->kind == NodeKind::ReduceScatter) {
        if (st->greduce && st->greduce != n) return *why = "more than one ReduceScatter", false;
        if (n->red != Summation || n->in[0]->kind != NodeKind::Tensor)
          return *why = "the ReduceScatter must sum a Local tensor", false;
        st->greduce = n;
        st->ggrad = n->in[0];
      }
      if (n->kind == NodeKind::Update && n->in[0]->layout == Replicated) {
        if (st->gweight) return *why = "more than one Replicated tensor is updated", false;
        if (n->in[1]->kind != NodeKind::AllGather) return *why = "the Replicated update is not an AllGather", false;
        st->gweight = n->in[0];
        st->gvalue = n->in[1]->in[0];
      }
      if (n->kind == NodeKind::Tensor && n->layout == Replicated && n->type != Float32)
        return *why = "Replicated tensors must be Float32", false;
    }
    if (!st->greduce) return *why = "no ReduceScatter", false;
    if (!st->gweight) return *why = "no AllGather into a Replicated tensor", false;
    if (st->ggrad->type != Float32 && st->ggrad->type != Float16)
      return *why = "gradients must be Float32 or Float16", false;
    return true;
  }

  // Expression inside the functor: i0 = index in the slice, gi = global index,
  // gsum = the reduced gradient element, w_old = the weight element.
  std::string fexpr(const Step &st, const NodeRef &n, const std::set<const Node *> &done) const {
    if (n.get() == st.greduce.get()) return "gsum";
    if (n->stage_id >= 0 && done.count(n.get())) {
      if (n->kind == NodeKind::Update) return n->in[0]->name + "[i0]";
      return n->name;
    }
    switch (n->kind) {
      case NodeKind::Const: return fmtConst(n->value, n->type);
      case NodeKind::Variable: return n->name;
      case NodeKind::Tensor:
        if (n.get() == st.gweight.get()) return "w_old";
        return n->layout == Sliced ? n->name + "[i0]" : n->name + "[gi]";
      case NodeKind::Binary:
        return "(" + fexpr(st, n->in[0], done) + " " + n->op + " " + fexpr(st, n->in[1], done) + ")";
      case NodeKind::Sqrt: return "sqrtf(" + fexpr(st, n->in[0], done) + ")";
      case NodeKind::Cast:
        return "((" + std::string(elemTypeName(n->type)) + ")" + fexpr(st, n->in[0], done) + ")";
      case NodeKind::Scatter:
      case NodeKind::AllGather: return fexpr(st, n->in[0], done);
      case NodeKind::Update: return n->in[0]->name + "[i0]";
      default: fail("cannot emit node inside a fused functor");
    }
  }

  // Members of the functor: Sliced tensors, other Replicated tensors, Variables.
  void functorMembers(const Step &st, std::vector<std::string> *decl, std::vector<std::string> *init) const {
    std::set<std::string> seen;
    std::function<void(const NodeRef &, bool)> walk = [&](const NodeRef &n, bool root) {
      if (!root && n->stage_id >= 0) {
        bool member = false;
        for (const NodeRef &s : st.stages) member = member || s.get() == n.get();
        if (!member) fail("a fused group reads stage " + n->name + " computed outside it");
        return;
      }
      if (n->kind == NodeKind::Variable && seen.insert(n->name).second) {
        decl->push_back(std::string(elemTypeName(n->type)) + " " + n->name);
        init->push_back(n->name);
      }
      if (n->kind == NodeKind::Tensor && n.get() != st.ggrad.get() && n.get() != st.gweight.get() &&
          seen.insert(n->name).second) {
        decl->push_back(std::string(elemTypeName(n->type)) + "* " + n->name);
        init->push_back(n->name);
      }
      for (const NodeRef &c : n->in) walk(c, false);
    };
    for (const NodeRef &s : st.stages) walk(s, true);
  }

  void emitFunctor(const Step &st) {
    std::vector<std::string> decl, init;
    functorMembers(st, &decl, &init);
    kernels << "// The arithmetic of the fused group, applied to one element of this rank's slice.\n";
    kernels << "struct " << p.name() << "Fused" << st.kernel_id << " {\n";
    for (const std::string &d : decl) kernels << "  " << d << ";\n";
    kernels << "  __device__ __forceinline__ float operator()(size_t i0, size_t gi, float gsum, float w_old) const {\n";
    kernels << "    (void)i0; (void)gi; (void)gsum; (void)w_old;\n";
    std::set<const Node *> done;
    std::string result = "w_old";
    for (const NodeRef &s : st.stages) {
      if (s.get() == st.greduce.get()) {
        done.insert(s.get());
        continue;
      }
      if (s->kind == NodeKind::Update) {
        if (s->in[0].get() == st.gweight.get()) {
          result = fexpr(st, s->in[1], done);
        } else {
          kernels << "    " << s->in[0]->name << "[i0] = " << fexpr(st, s->in[1], done) << ";\n";
        }
      } else {
        NodeRef tmp = std::make_shared<Node>(*s);
        tmp->stage_id = -1;
        kernels << "    " << elemTypeName(s->type) << " " << s->name << " = " << fexpr(st, tmp, done) << ";\n";
      }
      done.insert(s.get());
    }
    kernels << "    return " << result << ";\n  }\n};\n\n";
  }

  std::string genericCall(const Step &st) const {
    std::vector<std::string> decl, init;
    functorMembers(st, &decl, &init);
    std::ostringstream o;
    const std::string gt = st.ggrad->type == Float16 ? "__half" : "float";
    o << "  {\n    cocoGenericPlan plan;\n";
    o << "    COCOCHECK(cocoFusedGenericPlan(comm, " << st.ggrad->name << ", " << cocoType(st.ggrad->type)
      << ", " << st.gweight->name << ", " << N() << ", 1.0f, stream, &plan));\n";
    o << "    " << p.name() << "Fused" << st.kernel_id << " f = {";
    for (size_t k = 0; k < init.size(); ++k) o << (k ? ", " : "") << init[k];
    o << "};\n";
    o << "    COCOCHECK(cocoLaunchGenericFused<" << gt << ">(plan, f, stream));\n  }\n";
    return o.str();
  }

  // ---- expressions inside a generated kernel ----------------------------------
  // `sliced_space`: the kernel iterates over the rank's slice; Replicated and
  // Local tensors are then addressed at slice_start + i0.
  std::string tensorRef(const NodeRef &t, bool sliced_space) const {
    if (t->layout == Sliced || !sliced_space) return t->name + "[i0]";
    return t->name + "[" + sliceCount() + " * rank + i0]";
  }

  std::string expr(const NodeRef &n, bool sliced_space, const std::set<const Node *> &local) const {
    // a stage computed earlier in this kernel: its register, unless it lives in memory
    if (n->stage_id >= 0 && local.count(n.get()) && n->kind != NodeKind::Update &&
        !buffer.count(n.get()))
      return n->name;
    if (n->stage_id >= 0 && n->kind != NodeKind::Update && !isCollective(n->kind) &&
        buffer.count(n.get())) {
      if (n->scalar) return "(*" + buffer.at(n.get()) + ")";
      return buffer.at(n.get()) + (n->layout == Sliced || !sliced_space
                                       ? "[i0]"
                                       : "[" + sliceCount() + " * rank + i0]");
    }
    switch (n->kind) {
      case NodeKind::Const: return fmtConst(n->value, n->type);
      case NodeKind::Variable: return n->name;
      case NodeKind::Tensor: return tensorRef(n, sliced_space);
      case NodeKind::Binary:
        return "(" + expr(n->in[0], sliced_space, local) + " " + n->op + " " +
               expr(n->in[1], sliced_space, local) + ")";
      case NodeKind::Sqrt: return "sqrtf(" + expr(n->in[0], sliced_space, local) + ")";
      case NodeKind::Cast:
        return "((" + std::string(elemTypeName(n->type)) + ")" + expr(n->in[0], sliced_space, local) + ")";
      case NodeKind::Scatter: {
        const NodeRef &t = n->in[0];
        if (t->kind == NodeKind::Tensor) return t->name + "[" + sliceCount() + " * rank + i0]";
        return expr(t, sliced_space, local);
      }
      case NodeKind::Update:  // value of an updated tensor = the tensor's new contents
        return tensorRef(n->in[0], sliced_space);
      case NodeKind::AllReduce:  // reduced in place in the gradient buffer
        return tensorRef(n->in[0], sliced_space);
      case NodeKind::ReduceScatter:
        return n->in[0]->name + "[" + sliceCount() + " * rank + i0]";
      case NodeKind::AllGather: return expr(n->in[0], sliced_space, local);
      default: fail("cannot emit node inside a kernel");
    }
  }

  // Tensors, variables and buffers a kernel step reads or writes.
  void kernelParams(const Step &st, std::vector<std::string> *decl, std::vector<std::string> *call) const {
    std::set<std::string> seen;
    auto add = [&](const std::string &type, const std::string &name) {
      if (seen.insert(name).second) {
        decl->push_back(type + " " + name);
        call->push_back(name);
      }
    };
    add("size_t", N());
    std::set<const Node *> local;
    for (const NodeRef &s : st.stages) local.insert(s.get());
    std::function<void(const NodeRef &, bool)> walk = [&](const NodeRef &n, bool root) {
      if (!root && n->stage_id >= 0 && !local.count(n.get())) {
        if (n->kind == NodeKind::Update) add(std::string(elemTypeName(n->type)) + "*", n->in[0]->name);
        else if (isCollective(n->kind)) {
          NodeRef t = n->in[0];
          while (t->kind != NodeKind::Tensor && !t->in.empty()) t = t->in[0];
          add(std::string(elemTypeName(t->type)) + "*", t->name);
        } else if (buffer.count(n.get()))
          add(std::string(elemTypeName(n->type)) + "*", buffer.at(n.get()));
        return;
      }
      if (!root && n->stage_id >= 0) return;
      if (n->kind == NodeKind::Variable) add(elemTypeName(n->type), n->name);
      if (n->kind == NodeKind::Tensor) add(std::string(elemTypeName(n->type)) + "*", n->name);
      for (const NodeRef &c : n->in) walk(c, false);
    };
    for (const NodeRef &s : st.stages) {
      walk(s, true);
      if (buffer.count(s.get())) add(std::string(elemTypeName(s->type)) + "*", buffer.at(s.get()));
    }
    add("int", "comm_size");
    add("int", "rank");
  }

  bool slicedSpace(const Step &st) const {
    for (const NodeRef &s : st.stages)
      if (s->layout == Sliced) return true;
    return false;
  }

  void emitKernel(const Step &st) {
    std::vector<std::string> decl, call;
    kernelParams(st, &decl, &call);
    const bool sliced = slicedSpace(st);
    kernels << "__global__ void " << st.label << "(";
    for (size_t k = 0; k < decl.size(); ++k) kernels << (k ? ", " : "") << decl[k];
    kernels << ") {\n";
    kernels << "  size_t i0 = threadIdx.x + (size_t)blockDim.x * blockIdx.x;\n";
    if (sliced) {
      kernels << "  size_t __lo = (size_t)" << sliceCount() << " * rank;\n";
      kernels << "  if (__lo + i0 >= " << N() << " || i0 >= " << sliceCount() << ") return;\n";
    } else {
      kernels << "  if (i0 >= " << N() << ") return;\n";
    }
    std::set<const Node *> local;
    for (const NodeRef &s : st.stages) {
      const std::string ty = elemTypeName(s->type);
      if (s->kind == NodeKind::Update) {
        kernels << "  " << tensorRef(s->in[0], sliced) << " = " << expr(s->in[1], sliced, local) << ";\n";
      } else {
        // evaluate the stage's own expression (not a reference to itself)
        std::string rhs;
        {
          std::set<const Node *> l2 = local;
          NodeRef tmp = std::make_shared<Node>(*s);
          tmp->stage_id = -1;
          rhs = expr(tmp, sliced, l2);
        }
        if (buffer.count(s.get()))
          kernels << "  " << buffer.at(s.get()) << "[i0] = " << rhs << ";\n";
        else
          kernels << "  " << ty << " " << s->name << " = " << rhs << ";\n";
      }
      local.insert(s.get());
    }
    kernels << "}\n\n";
  }

  // ---- the step function --------------------------------------------------------
  std::vector<std::string> intermediates() const {  // declaration order = stage order
    std::vector<std::string> out;
    for (const NodeRef &s : p.stages())
      if (buffer.count(s.get())) out.push_back(buffer.at(s.get()));
    return out;
  }
  const Node *stageByBuffer(const std::string &b) const {
    for (const auto &kv : buffer)
      if (kv.second == b) return kv.first;
    return nullptr;
  }

  void emitTimed(std::ostream &os, const std::string &label, const std::string &body) const {
    os << "  CUDACHECK(cudaEventRecord(start" << p.name() << ", stream));\n";
    os << body;
    os << "  CUDACHECK(cudaEventRecord(stop" << p.name() << ", stream));\n";
    os << "  CUDACHECK(cudaEventSynchronize(stop" << p.name() << "));\n";
    os << "  CUDACHECK(cudaEventElapsedTime(&elapsedTime, start" << p.name() << ", stop" << p.name() << "));\n";
    os << "  elapsedTime" << label << " += elapsedTime;\n\n";
  }

  std::string fusedCall(const FusedUpdate &fu) const {
    auto orOne = [](const std::string &v) { return v.empty() ? std::string("1.0f") : v; };
    std::ostringstream c;
    const std::string gt = cocoType(fu.grad->type);
    if (fu.weight->type != Float32) fail("the fused step keeps fp32 weights ('" + fu.weight->name + "')");
    // Mixed precision (the reference's hook passes `(half*)g, w, (half*)w`,
    // src/codegen.cpp:1910): the 16-bit Replicated copy is what is gathered; the
    // fp32 master is a Sliced tensor, which the runtime indexes by GLOBAL element
    // inside the rank's slice only -- hence the pointer moved back by the slice
    // start.
    std::string w = fu.weight->name, lp = "NULL", lpt = "cocoFloat16";
    if (fu.lp) {
      if (fu.weight->layout != Sliced) fail("mixed precision: the fp32 master '" + w + "' must be Sliced");
      w = "(" + w + " - (size_t)" + sliceCount() + " * rank)";
      lp = fu.lp->name;
      lpt = cocoType(fu.lp->type);
    }
    const std::string gs = fu.gscale.empty() ? std::string("1.0f")
                           : fu.gscale_div ? "(1.0f / " + fu.gscale + ")" : fu.gscale;
    switch (fu.rule) {
      case FusedUpdate::SGD:
        c << "cocoFusedSGD(comm, " << fu.grad->name << ", " << gt << ", " << w << ", " << lp << ", "
          << lpt << ", " << N() << ", " << orOne(fu.lr) << ", " << gs << ", stream)";
        break;
      case FusedUpdate::Adam:
        c << "cocoFusedAdam(comm, " << fu.grad->name << ", " << gt << ", " << w << ", " << lp << ", "
          << lpt << ", " << fu.m->name << ", " << fu.v->name << ", " << N() << ", "
          << orOne(fu.lr) << ", " << fu.beta1 << ", " << fu.beta2
          << ", 0.0f, iter, " << gs << ", cocoVariantDsl, stream)";
        break;
      case FusedUpdate::LAMB:
        c << "cocoFusedLAMB(comm, " << fu.grad->name << ", " << gt << ", " << w << ", " << lp << ", "
          << lpt << ", " << fu.m->name << ", " << fu.v->name << ", " << N() << ", "
          << orOne(fu.lr) << ", " << fu.beta1 << ", " << fu.beta2 << ", 0.0f, "
          << (fu.decay.empty() ? std::string("0.0f") : fu.decay)
          << ", iter, " << gs << ", cocoVariantDsl, 0, stream)";
        break;
      default: fail("unclassified fused group");
    }
    return c.str();
  }

  std::string collectiveCall(const Step &st) const {
    const NodeRef &c = st.coll;
    std::ostringstream o;
    NodeRef src = c->in[0];
    // the value being communicated lives in a tensor, an Update target or a buffer
    auto memName = [&](const NodeRef &n) -> std::string {
      if (n->kind == NodeKind::Tensor) return n->name;
      if (n->kind == NodeKind::Update) return n->in[0]->name;
      if (buffer.count(n.get())) return buffer.at(n.get());
      fail("operand of a collective is not in memory: " + n->name);
    };
    const std::string in = memName(src);
    const bool own = c->type == Float32 && c->kind != NodeKind::Broadcast &&
                     (c->kind == NodeKind::AllGather || c->red == Summation);
    if (own) {  // the runtime's collectives on peer memory: no NCCL in the program
      if (c->kind == NodeKind::AllReduce) {
        o << "  COCOCHECK(cocoAllReduce(comm, " << in << ", " << N() << ", stream));\n";
      } else if (c->kind == NodeKind::ReduceScatter) {  // in place: the own slice of the own buffer
        o << "  COCOCHECK(cocoReduceScatter(comm, " << in << ", " << in << " + (size_t)" << sliceCount()
          << " * rank, " << N() << ", stream));\n";
      } else {
        const NodeRef &stage = st.stages[0];
        if (stage->kind != NodeKind::Update) fail("AllGather result must Update a Replicated tensor");
        o << "  COCOCHECK(cocoAllGather(comm, " << in << ", " << stage->in[0]->name << ", " << N()
          << ", stream));\n";
      }
      return o.str();
    }
    const std::string ty = ncclType(c->type);
    if (c->kind == NodeKind::AllReduce) {
      o << "  NCCLCHECK(ncclAllReduce(" << in << ", " << in << ", " << N() << ", " << ty
        << ", ncclSum, nccl, stream));\n";
    } else if (c->kind == NodeKind::ReduceScatter) {  // in place: slice r of every rank's buffer
      o << "  NCCLCHECK(ncclReduceScatter(" << in << ", " << in << " + (size_t)" << sliceCount()
        << " * rank, " << sliceCount() << ", " << ty << ", ncclSum, nccl, stream));\n";
    } else if (c->kind == NodeKind::AllGather) {
      const NodeRef &stage = st.stages[0];
      if (stage->kind != NodeKind::Update) fail("AllGather result must Update a Replicated tensor");
      o << "  NCCLCHECK(ncclAllGather(" << in << ", " << stage->in[0]->name << ", " << sliceCount()
        << ", " << ty << ", nccl, stream));\n";
    } else {
      fail("Broadcast is not emitted yet");
    }
    return o.str();
  }

  std::string normCalls(const Step &st) const {
    const NodeRef &nrm = st.stages[0];
    const NodeRef &x = nrm->in[0];
    std::string src, count;
    if (x->kind == NodeKind::Tensor) src = x->name;
    else if (x->kind == NodeKind::Update) src = x->in[0]->name;
    else if (buffer.count(x.get())) src = buffer.at(x.get());
    else if (x->kind == NodeKind::AllReduce || x->kind == NodeKind::ReduceScatter) {
      // the collectives work in place: the sum is in the operand's own memory
      // (a reduce-scatter leaves it in the rank's slice of that memory)
      const NodeRef &t = x->in[0];
      std::string mem = t->kind == NodeKind::Tensor ? t->name
                        : t->kind == NodeKind::Update ? t->in[0]->name
                        : buffer.count(t.get()) ? buffer.at(t.get()) : "";
      if (mem.empty()) fail("operand of Norm is not in memory: " + x->name);
      src = x->kind == NodeKind::AllReduce ? mem : "(" + mem + " + (size_t)" + sliceCount() + " * rank)";
    }
    else fail("operand of Norm is not in memory: " + x->name);
    const bool sliced = x->layout == Sliced;
    count = sliced ? "coconetSliceLen(" + N() + ", comm_size, rank)" : N();
    std::ostringstream o;
    const std::string acc = buffer.at(nrm.get()) + "_acc";
    o << "  CUDACHECK(cudaMemsetAsync(" << acc << ", 0, sizeof(double), stream));\n";
    o << "  coconetSumSquares<<<coconetBlocks(" << count << "), 256, 0, stream>>>(" << src << ", "
      << count << ", " << acc << ");\n";
    if (sliced)  // the partial sums of the ranks' slices meet on the host (8 bytes per rank)
      o << "  coconetSumOverRanks(comm, " << acc << ", stream);\n";
    o << "  coconetFinishNorm<<<1, 1, 0, stream>>>(" << acc << ", " << buffer.at(nrm.get()) << ");\n";
    return o.str();
  }

  // ---- host reference of one step (the reference's mpiRef idea, src/codegen.cpp:
  // 4421-4581, which its own generator leaves disabled): every stage evaluated
  // per element on the host in float, from the tensors' initial values.  The
  // generated programs give every rank the same inputs, so the reduced
  // gradient is the rank-order sum of comm_size equal values and the global
  // view of a Sliced tensor is its per-rank array repeated.
  std::string hostExpr(const NodeRef &n, bool root) const {
    if (!root && n->stage_id >= 0) return n->scalar ? "v_" + n->name : "v_" + n->name + "[i0]";
    switch (n->kind) {
      case NodeKind::Const: return fmtConst(n->value, Float32);
      case NodeKind::Variable: return n->name;
      case NodeKind::Tensor:
        return n->layout == Sliced ? "h_" + n->name + "[i0 % S]" : "h_" + n->name + "[i0]";
      case NodeKind::Binary:
        return "(" + hostExpr(n->in[0], false) + " " + n->op + " " + hostExpr(n->in[1], false) + ")";
      case NodeKind::Sqrt: return "sqrtf(" + hostExpr(n->in[0], false) + ")";
      case NodeKind::Cast:  // values are held as float on the host: a cast to half rounds
        return n->type == Float16 ? "coconetRoundHalf(" + hostExpr(n->in[0], false) + ")"
                                  : "((float)" + hostExpr(n->in[0], false) + ")";
      case NodeKind::Scatter:
      case NodeKind::AllGather:
      case NodeKind::Broadcast: return hostExpr(n->in[0], false);
      case NodeKind::Update: return hostExpr(n->in[1], false);
      case NodeKind::AllReduce:
      case NodeKind::ReduceScatter:
        return "coconetRankSum(" + hostExpr(n->in[0], false) + ", comm_size)";
      default: fail("cannot emit node in the host reference");
    }
  }

  // a 16-bit tensor may differ from the host's rounding by one unit in its last place
  static std::string closeFn(const NodeRef &t) {
    return t->type == Float16 ? "coconetCloseHalf" : "coconetClose";
  }

  void emitHostRef(std::ostream &os) const {
    os << "// Host evaluation of one step of pipeline '" << p.name() << "' (iteration 0).\n";
    os << "static bool hostRef(size_t " << N() << ", int comm_size, int rank";
    for (const NodeRef &a : args) {
      if (a->kind == NodeKind::Variable) os << ", float " << a->name;
      else os << ", const std::vector<float>& h_" << a->name << ", const std::vector<float>& d_" << a->name;
    }
    os << ") {\n";
    os << "  const size_t S = DIVUP(" << N() << ", (size_t)comm_size);\n";
    os << "  const size_t lo = S * rank < " << N() << " ? S * rank : " << N() << ";\n";
    os << "  const size_t len = lo + S < " << N() << " ? S : " << N() << " - lo;\n";
    for (const NodeRef &s : p.stages()) {
      if (s->kind == NodeKind::Norm) {
        os << "  float v_" << s->name << ";\n  {\n    double acc = 0.0;\n"
           << "    for (size_t i0 = 0; i0 < " << N() << "; i0++) { double x = " << hostExpr(s->in[0], false)
           << "; acc += x * x; }\n    v_" << s->name << " = (float)sqrt(acc);\n  }\n";
      } else if (s->scalar) {
        os << "  float v_" << s->name << " = " << hostExpr(s, true) << ";\n";
      } else {
        os << "  std::vector<float> v_" << s->name << "(" << N() << ");\n";
        os << "  for (size_t i0 = 0; i0 < " << N() << "; i0++) v_" << s->name << "[i0] = "
           << hostExpr(s, true) << ";\n";
      }
    }
    os << "  bool ok = true;\n";
    for (const NodeRef &s : p.stages()) {
      if (s->kind != NodeKind::Update) continue;
      const NodeRef &t = s->in[0];
      if (t->layout == Sliced) {
        os << "  for (size_t j = 0; j < len && ok; j++)\n"
           << "    if (!" << closeFn(t) << "(v_" << s->name << "[lo + j], d_" << t->name << "[j])) {\n"
           << "      printf(\"rank %d: mismatch in " << t->name << "[%ld]: ref %g, computed %g\\n\", rank, (long)j, v_"
           << s->name << "[lo + j], d_" << t->name << "[j]);\n      ok = false;\n    }\n";
      } else {
        os << "  for (size_t i0 = 0; i0 < " << N() << " && ok; i0++)\n"
           << "    if (!" << closeFn(t) << "(v_" << s->name << "[i0], d_" << t->name << "[i0])) {\n"
           << "      printf(\"rank %d: mismatch in " << t->name << "[%ld]: ref %g, computed %g\\n\", rank, (long)i0, v_"
           << s->name << "[i0], d_" << t->name << "[i0]);\n      ok = false;\n    }\n";
      }
    }
    os << "  return ok;\n}\n\n";
  }

  // ---- whole program ---------------------------------------------------------------
  void emit(std::ostream &os) {
    plan();
    // Norm results need a buffer even when only read in the next kernel
    for (const Step &st : steps)
      if (st.kind == Step::NormReduce) buffer[st.stages[0].get()] = st.stages[0]->name;
    bool has_generic = false;
    for (const Step &st : steps) {
      if (st.kind == Step::Kernel) emitKernel(st);
      if (st.kind == Step::FusedGeneric) {
        emitFunctor(st);
        has_generic = true;
      }
    }

    os << "// Generated by the coconet-b200 DSL emitter from pipeline '" << p.name() << "'.\n";
    if (needs_nccl) os << "#define COCONET_USE_NCCL 1\n";
    os << "#include \"header.h\"\n";
    if (has_generic) os << "#include \"coconet_fused_generic.cuh\"\n";
    os << "\n" << kernels.str();

    // signature
    std::vector<std::string> decl, call;
    decl.push_back("size_t " + N());
    call.push_back(N());
    for (const NodeRef &a : args) {
      if (a->kind == NodeKind::Variable) {
        decl.push_back(std::string(elemTypeName(a->type)) + " " + a->name);
      } else {
        decl.push_back(std::string(elemTypeName(a->type)) + "* " + a->name);
      }
      call.push_back(a->name);
    }
    for (const std::string &b : intermediates()) {
      const Node *s = stageByBuffer(b);
      decl.push_back(std::string(elemTypeName(s->type)) + "* " + b);
      call.push_back(b);
      if (s->kind == NodeKind::Norm) {
        decl.push_back("double* " + b + "_acc");
        call.push_back(b + "_acc");
      }
    }
    decl.push_back("int iter");
    call.push_back("iter");
    std::vector<std::string> labels;
    for (const Step &st : steps) {
      labels.push_back(st.label);
      decl.push_back("float& elapsedTime" + st.label);
      call.push_back("elapsedTime" + st.label);
    }
    decl.push_back("cocoComm_t comm");
    call.push_back("comm");
    if (needs_nccl) {
      decl.push_back("ncclComm_t nccl");
      call.push_back("nccl");
    }
    decl.push_back("cudaStream_t stream");
    call.push_back("stream");
    decl.push_back("int comm_size");
    call.push_back("comm_size");
    decl.push_back("int rank");
    call.push_back("rank");

    // the host evaluation holds every value as float: programs over fp32 and fp16
    bool all_float = true;
    for (const NodeRef &a : args)
      all_float = all_float && (a->type == Float32 || (a->type == Float16 && a->kind == NodeKind::Tensor));
    if (all_float) emitHostRef(os);

    os << "void " << p.name() << "(";
    for (size_t k = 0; k < decl.size(); ++k) os << (k ? ", " : "") << decl[k];
    os << ") {\n";
    os << "  cudaEvent_t start" << p.name() << ", stop" << p.name() << ";\n";
    os << "  float elapsedTime;\n";
    os << "  CUDACHECK(cudaEventCreate(&start" << p.name() << "));\n";
    os << "  CUDACHECK(cudaEventCreate(&stop" << p.name() << "));\n\n";
    for (const Step &st : steps) {
      std::ostringstream body;
      switch (st.kind) {
        case Step::Fused:
          body << "  COCOCHECK(" << fusedCall(st.fused) << ");\n";
          break;
        case Step::FusedGeneric:
          body << genericCall(st);
          break;
        case Step::Collective:
          body << collectiveCall(st);
          break;
        case Step::NormReduce:
          body << normCalls(st);
          break;
        case Step::Kernel: {
          std::vector<std::string> kd, kc;
          kernelParams(st, &kd, &kc);
          const std::string total = slicedSpace(st) ? sliceCount() : N();
          body << "  {\n    size_t totalThreads = (size_t)" << total << ";\n"
               << "    size_t numThreads = totalThreads < 256 ? totalThreads : 256;\n"
               << "    size_t numThreadBlocks = DIVUP(totalThreads, numThreads);\n"
               << "    " << st.label << "<<<numThreadBlocks, numThreads, 0, stream>>>(";
          for (size_t k = 0; k < kc.size(); ++k) body << (k ? ", " : "") << kc[k];
          body << ");\n  }\n";
          break;
        }
      }
      emitTimed(os, st.label, body.str());
    }
    os << "  CUDACHECK(cudaEventDestroy(start" << p.name() << "));\n";
    os << "  CUDACHECK(cudaEventDestroy(stop" << p.name() << "));\n";
    os << "}\n\n";

    // main
    os << "int main(int argc, char** argv) {\n";
    os << "  // usage: prog <epochs> [first log2 size = 10] [last log2 size (exclusive) = 30] [check]\n";
    os << "  int N_GPUs;\n  CUDACHECK(cudaGetDeviceCount(&N_GPUs));\n";
    os << "  int comm_size, rank, local_rank;\n";
    os << "  COCOCHECK(cocoEnvRank(&rank, &comm_size, &local_rank));\n";
    os << "  CUDACHECK(cudaSetDevice(local_rank % N_GPUs));\n";
    os << "  cocoComm_t comm;\n";
    os << "  COCOCHECK(cocoCommInitRank(&comm, comm_size, rank, NULL));\n";
    if (needs_nccl) os << "  ncclComm_t nccl = coconetNcclInit(comm, comm_size, rank);\n";
    os << "  if (argc < 2) { printf(\"Specify epochs as command arg\\n\"); return 1; }\n";
    os << "  int epochs = atoi(argv[1]);\n";
    os << "  int firstLog = argc > 2 ? atoi(argv[2]) : 10;\n";
    os << "  int lastLog = argc > 3 ? atoi(argv[3]) : 30;\n";
    os << "  bool check = argc > 4 && std::string(argv[4]) == \"check\";\n";
    os << "  cudaStream_t stream;\n  CUDACHECK(cudaStreamCreate(&stream));\n";
    os << "  COCOCHECK(cocoBarrier(comm));\n\n";
    os << "  for (int __i = firstLog; __i < lastLog; __i++) {\n";
    os << "    size_t " << N() << " = 1UL << __i;\n";
    os << "    // Inputs\n";
    // Buffers the fused step lets peers touch come from the runtime's symmetric
    // allocator (peer mappings + NVSwitch multicast where the node has it).
    std::set<const Node *> symmetric;
    for (const Step &st : steps) {
      if (st.kind == Step::Fused) {  // what peers read (gradients) and write (the gathered tensor)
        symmetric.insert(st.fused.grad.get());
        symmetric.insert(st.fused.lp ? st.fused.lp.get() : st.fused.weight.get());
      }
      if (st.kind == Step::FusedGeneric) {
        symmetric.insert(st.ggrad.get());
        symmetric.insert(st.gweight.get());
      }
      if (st.kind == Step::Collective) {  // what peers read (the reduced tensor) or write (the gathered one)
        const NodeRef &src = st.coll->in[0];
        if (src->kind == NodeKind::Tensor) symmetric.insert(src.get());
        if (st.stages[0]->kind == NodeKind::Update) symmetric.insert(st.stages[0]->in[0].get());
      }
    }
    std::vector<std::string> frees, symm_frees;
    for (const NodeRef &a : args) {
      const std::string ty = elemTypeName(a->type);
      if (a->kind == NodeKind::Variable) {
        // 1.0f as in the reference's generated programs; COCONET_SCALAR_<name> overrides
        os << "    " << ty << " " << a->name << ";\n    " << a->name << " = coconetScalar(\"" << a->name
           << "\", 1.0f);\n";
      } else {
        // Sliced tensors hold DIVUP(N, comm_size) elements (reference: genNumElem,
        // src/codegen.cpp:139-165)
        const std::string cnt = a->layout == Sliced ? sliceCount() : N();
        os << "    " << ty << "* " << a->name << ";\n";
        if (symmetric.count(a.get())) {
          os << "    COCOCHECK(cocoMemAlloc(comm, (void**)&" << a->name << ", " << cnt << " * sizeof(" << ty
             << ")));\n";
          symm_frees.push_back(a->name);
        } else {
          os << "    CUDACHECK(cudaMalloc(&" << a->name << ", " << cnt << " * sizeof(" << ty << ")));\n";
          frees.push_back(a->name);
        }
        os << "    cudaMemRandInt(" << a->name << ", " << cnt << ");\n";
      }
    }
    os << "\n    // Intermediates\n";
    for (const std::string &b : intermediates()) {
      const Node *s = stageByBuffer(b);
      const std::string ty = elemTypeName(s->type);
      const std::string cnt = s->scalar ? "1" : (s->layout == Sliced ? sliceCount() : N());
      os << "    " << ty << "* " << b << ";\n";
      os << "    CUDACHECK(cudaMalloc(&" << b << ", " << cnt << " * sizeof(" << ty << ")));\n";
      frees.push_back(b);
      if (s->kind == NodeKind::Norm) {
        os << "    double* " << b << "_acc;\n";
        os << "    CUDACHECK(cudaMalloc(&" << b << "_acc, sizeof(double)));\n";
        frees.push_back(b + "_acc");
      }
    }
    for (const std::string &l : labels) os << "    float elapsedTime" << l << " = 0;\n";
    if (all_float) {
      os << "    if (check) {  // one step, compared with the host evaluation of the same pipeline\n";
      for (const NodeRef &a : args)
        if (a->kind == NodeKind::Tensor) {
          const std::string cnt = a->layout == Sliced ? sliceCount() : N();
          os << "      std::vector<float> h_" << a->name << "(" << cnt << "), d_" << a->name << "(" << cnt << ");\n";
          os << "      coconetToHost(h_" << a->name << ", " << a->name << ", " << cnt << ");\n";
        }
      os << "      { int iter = 0; " << p.name() << "(";
      for (size_t k = 0; k < call.size(); ++k) os << (k ? ", " : "") << call[k];
      os << "); }\n";
      os << "      CUDACHECK(cudaStreamSynchronize(stream));\n";
      os << "      coconetCheckStatus(comm, rank);\n";
      for (const NodeRef &a : args)
        if (a->kind == NodeKind::Tensor) {
          const std::string cnt = a->layout == Sliced ? sliceCount() : N();
          os << "      coconetToHost(d_" << a->name << ", " << a->name << ", " << cnt << ");\n";
        }
      os << "      bool pass = hostRef(" << N() << ", comm_size, rank";
      for (const NodeRef &a : args) {
        if (a->kind == NodeKind::Variable) os << ", " << a->name;
        else os << ", h_" << a->name << ", d_" << a->name;
      }
      os << ");\n";
      os << "      printf(\"rank %d: check of " << p.name() << " at SZ %ld %s\\n\", rank, (long)" << N()
         << ", pass ? \"PASSED\" : \"FAILED\");\n";
      os << "      if (!pass) exit(EXIT_FAILURE);\n";
      os << "      COCOCHECK(cocoBarrier(comm));\n";
      for (const std::string &l : labels) os << "      elapsedTime" << l << " = 0;\n";
      os << "    }\n";
    }
    // One untimed step first: the first launch of a kernel loads its module and,
    // across ranks, waits for the slowest process to get here.  (The reference's
    // frozen test programs skip their first iterations for the same reason,
    // examples/test-adam.cu:132-133.)
    os << "    if (!check) {\n      { int iter = 0; " << p.name() << "(";
    for (size_t k = 0; k < call.size(); ++k) os << (k ? ", " : "") << call[k];
    os << "); }\n      CUDACHECK(cudaStreamSynchronize(stream));\n";
    for (const std::string &l : labels) os << "      elapsedTime" << l << " = 0;\n";
    os << "    }\n";
    os << "    for (int iter = 1; iter <= epochs; iter++) {\n";
    os << "      " << p.name() << "(";
    for (size_t k = 0; k < call.size(); ++k) os << (k ? ", " : "") << call[k];
    os << ");\n    }\n";
    os << "    CUDACHECK(cudaStreamSynchronize(stream));\n";
    os << "    coconetCheckStatus(comm, rank);\n";
    os << "    COCOCHECK(cocoBarrier(comm));\n";
    for (const std::string &f : symm_frees) os << "    COCOCHECK(cocoMemFree(comm, " << f << "));\n";
    for (const std::string &f : frees) os << "    CUDACHECK(cudaFree(" << f << "));\n";
    os << "    if (rank == 0)\n      printf(\"{SZ: %ld, Epochs: %d";
    for (const std::string &l : labels) os << ", " << l << ": %f";
    os << ", Total: %f}\\n\", (long)" << N() << ", epochs";
    for (const std::string &l : labels) os << ", elapsedTime" << l;
    os << ", ";
    for (size_t k = 0; k < labels.size(); ++k) os << (k ? " + " : "") << "elapsedTime" << labels[k];
    os << ");\n";
    os << "  }\n";
    if (needs_nccl) os << "  ncclCommDestroy(nccl);\n";
    os << "  COCOCHECK(cocoCommDestroy(comm));\n";
    os << "  return 0;\n}\n";
  }
};

}  // namespace

void Pipeline::codegen(std::ostream &os) {
  Emitter e(*this, args_);
  e.emit(os);
}

}  // namespace ACCCDSL
