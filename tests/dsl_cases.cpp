// Host-side checks of the DSL: fusion validity (after the ideas of the
// reference's stale tests/fusion-test.cpp:9-83: base case, unused stage,
// three stages, cycle) and recognition of the fused update rule.  Prints one
// "name: result" line per case; tests/test_dsl.py compares them.
#include <dsl.hpp>
#include <pipeline.hpp>

#include <iostream>
#include <sstream>

using namespace ACCCDSL;

static const char *ruleName(FusedUpdate::Rule r) {
  switch (r) {
    case FusedUpdate::SGD: return "SGD";
    case FusedUpdate::Adam: return "Adam";
    case FusedUpdate::LAMB: return "LAMB";
    default: return "Unknown";
  }
}

int main() {
  Variable N(Int32, "N");
  Variable lr(Float32, "lr"), b1(Float32, "b1"), b2(Float32, "b2"), wd(Float32, "wd");
  {  // base case: two dependent pointwise stages
    Tensor g(Float32, N, Local, "g");
    Tensor w(Float32, N, Replicated, "w");
    Stage a = AllReduce(Summation, g);
    Stage b = a * lr;
    Stage c = Update(w, w - b);
    Pipeline p("base", {g, w, lr}, {c});
    std::cout << "base: " << p.canFuse({b.node(), c.node()}) << "\n";
    std::cout << "three: " << p.canFuse({a.node(), b.node(), c.node()}) << "\n";
    // a stage that is not part of the pipeline
    Stage stray = w * 2.0;
    std::cout << "unused: " << p.canFuse({b.node(), stray.node()}) << "\n";
    std::cout << "groups_before: " << p.groups().size() << "\n";
    p.fuse({b, c});
    std::cout << "groups_after: " << p.groups().size() << "\n";
  }
  {  // cycle: a -> b -> c and a -> c; fusing {a, c} would need b in the middle
    Tensor g(Float32, N, Local, "g");
    Tensor w(Float32, N, Replicated, "w");
    Stage s = AllReduce(Summation, g);
    Stage a = s * lr;
    Stage b = a + w;
    Stage c = Update(w, a - b);
    Pipeline p("cycle", {g, w, lr}, {c});
    std::string why;
    std::cout << "cycle: " << p.canFuse({a.node(), c.node()}, &why) << "\n";
    std::cout << "cycle_reason: " << (why.find("cycle") != std::string::npos) << "\n";
    std::cout << "cycle_all: " << p.canFuse({a.node(), b.node(), c.node()}) << "\n";
  }
  {  // SGD written with the operands the other way round, no learning rate
    Tensor g(Float32, N, Local, "g");
    Tensor w(Float32, N, Replicated, "w");
    Stage gs = ReduceScatter(Summation, g);
    Stage ws = (-1.0) * gs + Scatter(w);
    Stage wn = Update(w, AllGather(ws));
    Pipeline p("sgd2", {g, w}, {wn});
    FusedUpdate fu = p.classify({gs.node(), ws.node(), wn.node()});
    std::cout << "sgd_commuted: " << ruleName(fu.rule) << " lr='" << fu.lr << "'\n";
  }
  {  // Adam with the roles of the two Sliced tensors and variables permuted in the argument list
    Tensor g(Float32, N, Local, "grad");
    Tensor w(Float32, N, Replicated, "weights");
    Tensor sec(Float32, N, Sliced, "second");
    Tensor fst(Float32, N, Sliced, "first");
    Stage gs = ReduceScatter(Summation, g);
    Stage v1 = Update(sec, (1 - b2) * gs * gs + sec * b2);
    Stage m1 = Update(fst, fst * b1 + gs * (1 - b1));
    Stage ws = Scatter(w) - lr * (m1 / b1) / (v1 / b2);
    Stage wn = Update(w, AllGather(ws));
    Pipeline p("adam2", {g, w, sec, fst, b2, lr, b1}, {v1, m1, wn});
    FusedUpdate fu = p.classify({gs.node(), v1.node(), m1.node(), ws.node(), wn.node()});
    std::cout << "adam_permuted: " << ruleName(fu.rule) << " m=" << (fu.m ? fu.m->name : "") << " v="
              << (fu.v ? fu.v->name : "") << " b1=" << fu.beta1 << " b2=" << fu.beta2 << " lr=" << fu.lr
              << "\n";
  }
  {  // not an optimizer this runtime implements: momentum SGD with a sign flip
    Tensor g(Float32, N, Local, "g");
    Tensor w(Float32, N, Replicated, "w");
    Tensor m(Float32, N, Sliced, "m");
    Stage gs = ReduceScatter(Summation, g);
    Stage m1 = Update(m, b1 * m + gs);
    Stage ws = Scatter(w) + lr * m1;
    Stage wn = Update(w, AllGather(ws));
    Pipeline p("momentum", {g, w, m, lr, b1}, {m1, wn});
    FusedUpdate fu = p.classify({gs.node(), m1.node(), ws.node(), wn.node()});
    std::cout << "momentum: " << ruleName(fu.rule) << "\n";
  }
  return 0;
}
