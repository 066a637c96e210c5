// Pipeline: stage discovery, fusion groups, recognition of the fused update
// rule.  (What the reference does in src/pipeline.cpp:223-240, 298-426,
// 905-935 with visitors over its AST is done here on the node DAG.)
#include "pipeline.hpp"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <functional>
#include <random>

namespace ACCCDSL {

namespace {

[[noreturn]] void fail(const std::string &msg) {
  std::fprintf(stderr, "coconet pipeline: %s\n", msg.c_str());
  std::exit(1);
}

// Stages that stage `s` reads directly (walking through unnamed nodes).
void direct_deps(const NodeRef &n, bool root, std::vector<const Node *> *out) {
  if (!root && n->stage_id >= 0) {
    out->push_back(n.get());
    return;
  }
  for (const NodeRef &c : n->in) direct_deps(c, false, out);
}

}  // namespace

// All nodes owned by a stage: its expression tree down to (not including)
// other stages.
void ownedNodes(const NodeRef &n, bool root, std::vector<NodeRef> *out) {
  if (!root && n->stage_id >= 0) return;
  out->push_back(n);
  for (const NodeRef &c : n->in) ownedNodes(c, false, out);
}

Pipeline::Pipeline(const std::string &name, std::initializer_list<Expression> args,
                   std::initializer_list<Stage> outputs)
    : name_(name) {
  for (const Expression &a : args) {
    if (!a.node() || (a.node()->kind != NodeKind::Variable && a.node()->kind != NodeKind::Tensor))
      fail("pipeline '" + name + "': arguments must be Variables or Tensors");
    args_.push_back(a.node());
  }
  for (const Stage &s : outputs) outputs_.push_back(s.node());
  if (outputs_.empty()) fail("pipeline '" + name + "' has no outputs");

  rediscover();
}

void Pipeline::rediscover() {
  stages_.clear();
  // post-order DFS from the outputs = a topological order of the stages
  std::set<const Node *> seen;
  std::function<void(const NodeRef &)> visit = [&](const NodeRef &n) {
    if (!seen.insert(n.get()).second) return;
    for (const NodeRef &c : n->in) visit(c);
    if (n->stage_id >= 0) stages_.push_back(n);
    if ((n->kind == NodeKind::Variable || n->kind == NodeKind::Tensor)) {
      bool declared = false;
      for (const NodeRef &a : args_) declared = declared || a.get() == n.get();
      // the size Variable of a tensor need not be listed (the examples omit N)
      if (!declared && !(n->kind == NodeKind::Variable && n->type == Int32))
        fail("pipeline '" + name_ + "' uses '" + n->name + "' which is not among its arguments");
    }
  };
  for (const NodeRef &o : outputs_) visit(o);
}

bool Pipeline::canFuse(const std::vector<NodeRef> &stages, std::string *why) const {
  auto say = [&](const std::string &m) {
    if (why) *why = m;
    return false;
  };
  if (stages.empty()) return say("empty fusion set");
  std::set<const Node *> members;
  for (const NodeRef &s : stages) {
    if (!s || s->stage_id < 0) return say("not a stage");
    if (std::find(stages_.begin(), stages_.end(), s) == stages_.end())
      return say("stage " + s->name + " is not part of pipeline '" + name_ + "'");
    members.insert(s.get());
  }
  // include stages already fused with any member
  for (const auto &g : fused_) {
    bool touches = false;
    for (const Node *m : members) touches = touches || g.count(m);
    if (touches) members.insert(g.begin(), g.end());
  }
  // transitive dependencies between stages
  std::map<const Node *, std::set<const Node *>> deps;
  for (const NodeRef &s : stages_) {  // topological: deps of deps are complete
    std::vector<const Node *> d;
    direct_deps(s, true, &d);
    for (const Node *x : d) {
      deps[s.get()].insert(x);
      deps[s.get()].insert(deps[x].begin(), deps[x].end());
    }
  }
  // A stage outside the set that both depends on a member and is depended on
  // by a member would have to run in the middle of the fused kernel.
  for (const NodeRef &x : stages_) {
    if (members.count(x.get())) continue;
    bool uses_member = false, used_by_member = false;
    for (const Node *m : members) {
      uses_member = uses_member || deps[x.get()].count(m);
      used_by_member = used_by_member || deps[m].count(x.get());
    }
    if (uses_member && used_by_member)
      return say("fusing would create a cycle through stage " + x->name);
  }
  return true;
}

void Pipeline::fuse(std::initializer_list<Stage> stages) { fuse(std::vector<Stage>(stages)); }

void Pipeline::fuse(const std::vector<Stage> &stages) {
  std::vector<NodeRef> v;
  for (const Stage &s : stages) v.push_back(s.node());
  std::string why;
  if (!canFuse(v, &why)) fail("invalid fuse in pipeline '" + name_ + "': " + why);
  std::set<const Node *> merged;
  for (const NodeRef &s : v) merged.insert(s.get());
  for (auto it = fused_.begin(); it != fused_.end();) {
    bool touches = false;
    for (const Node *m : merged) touches = touches || it->count(m);
    if (touches) {
      merged.insert(it->begin(), it->end());
      it = fused_.erase(it);
    } else {
      ++it;
    }
  }
  fused_.push_back(merged);
}

std::vector<std::vector<NodeRef>> Pipeline::groups() const {
  // group id per stage
  std::map<const Node *, int> gid;
  std::vector<std::vector<NodeRef>> groups;
  for (const NodeRef &s : stages_) {
    if (gid.count(s.get())) continue;
    const std::set<const Node *> *fs = nullptr;
    for (const auto &g : fused_)
      if (g.count(s.get())) fs = &g;
    std::vector<NodeRef> members;
    if (fs) {
      for (const NodeRef &t : stages_)
        if (fs->count(t.get())) members.push_back(t);
    } else {
      members.push_back(s);
    }
    for (const NodeRef &t : members) gid[t.get()] = (int)groups.size();
    groups.push_back(members);
  }
  // order the groups topologically (Kahn; ties by first stage)
  const int G = (int)groups.size();
  std::vector<std::set<int>> before(G);
  for (int g = 0; g < G; ++g)
    for (const NodeRef &s : groups[g]) {
      std::vector<const Node *> d;
      direct_deps(s, true, &d);
      for (const Node *x : d)
        if (gid[x] != g) before[g].insert(gid[x]);
    }
  std::vector<std::vector<NodeRef>> ordered;
  std::vector<bool> done(G, false);
  for (int round = 0; round < G; ++round) {
    int pick = -1;
    for (int g = 0; g < G && pick < 0; ++g) {
      if (done[g]) continue;
      bool ready = true;
      for (int b : before[g]) ready = ready && done[b];
      if (ready) pick = g;
    }
    if (pick < 0) fail("cyclic fusion groups in pipeline '" + name_ + "'");
    done[pick] = true;
    ordered.push_back(groups[pick]);
  }
  return ordered;
}

// ---------------------------------------------------------------------------
// Recognising the update rule of a fused group.
//
// The reference keys on pipeline.name() (src/codegen.cpp:1906-1917).  Here the
// group is evaluated as scalar arithmetic on random sample values -- a
// collective is the identity on one element of the summed gradient, a Norm is
// a free symbol -- and compared with the closed form of each rule under every
// assignment of the program's tensors and variables to the rule's roles.
// ---------------------------------------------------------------------------
namespace {

struct Probe {
  std::map<const Node *, double> leaf;   // Variables, Tensors, Norm symbols
  std::map<const Node *, double> memo;
  std::map<const Node *, double> updated;  // target tensor -> new value

  double eval(const NodeRef &n) {
    auto it = memo.find(n.get());
    if (it != memo.end()) return it->second;
    double r = 0;
    switch (n->kind) {
      case NodeKind::Const: r = n->value; break;
      case NodeKind::Variable:
      case NodeKind::Tensor:
      case NodeKind::Norm: r = leaf.at(n.get()); break;
      case NodeKind::Binary: {
        const double a = eval(n->in[0]), b = eval(n->in[1]);
        r = n->op == '+' ? a + b : n->op == '-' ? a - b : n->op == '*' ? a * b : a / b;
        break;
      }
      case NodeKind::Sqrt: r = std::sqrt(eval(n->in[0])); break;
      case NodeKind::Cast:
      case NodeKind::Scatter:
      case NodeKind::AllReduce:
      case NodeKind::ReduceScatter:
      case NodeKind::AllGather:
      case NodeKind::Broadcast: r = eval(n->in[0]); break;
      case NodeKind::Update:
        r = eval(n->in[1]);
        updated[n->in[0].get()] = r;
        break;
    }
    memo[n.get()] = r;
    return r;
  }
};

bool close(double a, double b) {
  return std::fabs(a - b) <= 1e-9 * std::max(1.0, std::max(std::fabs(a), std::fabs(b)));
}

}  // namespace

FusedUpdate Pipeline::classify(const std::vector<NodeRef> &group) const {
  FusedUpdate fu;
  std::vector<NodeRef> nodes;
  for (const NodeRef &s : group) ownedNodes(s, true, &nodes);

  std::vector<NodeRef> updates, norms;
  NodeRef reduce;
  for (const NodeRef &n : nodes) {
    if (n->kind == NodeKind::ReduceScatter || n->kind == NodeKind::AllReduce) {
      if (reduce && reduce != n) return fu;  // one gradient reduction per fused group
      reduce = n;
    }
    if (n->kind == NodeKind::Update) updates.push_back(n);
    if (n->kind == NodeKind::Norm) norms.push_back(n);
  }
  if (!reduce || reduce->red != Summation || reduce->in[0]->kind != NodeKind::Tensor) return fu;
  fu.grad = reduce->in[0];
  std::vector<NodeRef> state;
  NodeRef wupd;
  for (const NodeRef &u : updates) {
    if (u->in[0]->layout == Replicated) {
      if (wupd) return fu;
      wupd = u;
    } else {
      state.push_back(u);
    }
  }
  if (!wupd) return fu;
  fu.weight = wupd->in[0];

  std::vector<NodeRef> fvars;  // float Variables of the program
  for (const NodeRef &a : args_)
    if (a->kind == NodeKind::Variable && (a->type == Float32 || a->type == Float16 || a->type == Float64))
      fvars.push_back(a);

  // sample environments
  std::mt19937 rng(12345);
  std::uniform_real_distribution<double> U(0.3, 0.9);
  const int kSamples = 3;
  std::vector<Probe> probes(kSamples);
  for (Probe &p : probes) {
    for (const NodeRef &a : args_) p.leaf[a.get()] = U(rng);
    for (const NodeRef &n : norms) p.leaf[n.get()] = U(rng) + 1.0;
    for (const NodeRef &n : nodes)
      if (n->kind == NodeKind::Variable && !p.leaf.count(n.get())) p.leaf[n.get()] = 8.0;  // sizes
    for (const NodeRef &s : group) p.eval(s);
  }
  auto val = [&](const Probe &p, const NodeRef &n) { return p.leaf.at(n.get()); };
  auto opt = [&](const Probe &p, const NodeRef &n) { return n ? p.leaf.at(n.get()) : 1.0; };
  std::vector<NodeRef> with_absent = fvars;
  with_absent.push_back(nullptr);

  // Mixed precision: the gathered Replicated tensor is a 16-bit COPY of fp32
  // master weights that every rank keeps as a Sliced tensor.  The master is the
  // Sliced update whose new value is the one the copy receives (a Cast is the
  // identity on the sample values).
  if (fu.weight->type == Float16) {
    NodeRef master;
    for (const NodeRef &u : state) {
      bool same = u->in[0]->type == Float32;
      for (const Probe &p : probes)
        same = same && close(p.updated.at(u->in[0].get()), p.updated.at(fu.weight.get()));
      if (same) {
        if (master) return fu;  // ambiguous
        master = u;
      }
    }
    if (!master) return fu;  // 16-bit weights without an fp32 master: no kernel for that
    fu.lp = fu.weight;
    fu.weight = master->in[0];
    state.erase(std::find(state.begin(), state.end(), master));
  }

  // The gradient as the update uses it: the reduced sum itself, or the sum
  // times / divided by one Variable (the loss scale).
  struct GradForm {
    NodeRef var;
    bool div;
  };
  std::vector<GradForm> gforms = {{nullptr, false}};
  for (const NodeRef &s : fvars) {
    gforms.push_back({s, false});
    gforms.push_back({s, true});
  }
  auto geff = [&](const Probe &p, const GradForm &f) {
    const double g = val(p, fu.grad);
    return !f.var ? g : f.div ? g / val(p, f.var) : g * val(p, f.var);
  };
  auto note_scale = [&](const GradForm &f) {
    fu.gscale = f.var ? f.var->name : "";
    fu.gscale_div = f.div;
  };

  if (state.empty() && norms.empty()) {  // SGD: w' = w - lr * g
    for (const GradForm &gf : gforms)
      for (const NodeRef &lr : with_absent) {
        if (gf.var && gf.var == lr) continue;
        bool ok = true;
        for (const Probe &p : probes)
          ok = ok && close(p.updated.at(fu.weight.get()),
                           val(p, fu.weight) - opt(p, lr) * geff(p, gf));
        if (ok) {
          fu.rule = FusedUpdate::SGD;
          fu.lr = lr ? lr->name : "";
          note_scale(gf);
          // w - (lr * s) * g cannot be told from w - lr * (s * g): with both a
          // learning rate and a scale the first match (no scale) is kept
          return fu;
        }
      }
    return fu;
  }
  if (state.size() != 2) return fu;

  for (const GradForm &gf : gforms)
    for (int perm = 0; perm < 2; ++perm) {
      const NodeRef m = state[perm]->in[0], v = state[1 - perm]->in[0];
      for (const NodeRef &b1 : fvars)
        for (const NodeRef &b2 : fvars) {
          if (gf.var && (gf.var == b1 || gf.var == b2)) continue;
          bool moments_ok = true;
          for (const Probe &p : probes) {
            const double g = geff(p, gf);
            moments_ok = moments_ok &&
                         close(p.updated.at(m.get()), val(p, b1) * val(p, m) + (1 - val(p, b1)) * g) &&
                         close(p.updated.at(v.get()), val(p, b2) * val(p, v) + (1 - val(p, b2)) * g * g);
          }
          if (!moments_ok) continue;
          if (norms.empty()) {  // Adam as the DSL writes it: w - lr * (m'/b1) / (v'/b2)
            for (const NodeRef &lr : with_absent) {
              bool ok = true;
              for (const Probe &p : probes) {
                const double mh = p.updated.at(m.get()) / val(p, b1);
                const double vh = p.updated.at(v.get()) / val(p, b2);
                ok = ok && close(p.updated.at(fu.weight.get()), val(p, fu.weight) - opt(p, lr) * mh / vh);
              }
              if (ok) {
                fu.rule = FusedUpdate::Adam;
                fu.m = m, fu.v = v;
                fu.beta1 = b1->name, fu.beta2 = b2->name, fu.lr = lr ? lr->name : "";
                note_scale(gf);
                return fu;
              }
            }
          } else if (norms.size() == 2) {  // LAMB: r = m^/sqrt(v^) + decay*w; w - lr*(|w|/|r|)*r
            for (int np = 0; np < 2; ++np) {
              const NodeRef nw = norms[np], nr = norms[1 - np];
              for (const NodeRef &lr : with_absent)
                for (const NodeRef &wd : with_absent) {
                  bool ok = true;
                  for (Probe &p : probes) {
                    const double mh = p.updated.at(m.get()) / (1 - val(p, b1));
                    const double vh = p.updated.at(v.get()) / (1 - val(p, b2));
                    const double r = mh / std::sqrt(vh) + opt(p, wd) * val(p, fu.weight);
                    ok = ok && close(p.eval(nr->in[0]), r) && close(p.eval(nw->in[0]), val(p, fu.weight)) &&
                         close(p.updated.at(fu.weight.get()),
                               val(p, fu.weight) - opt(p, lr) * (val(p, nw) / val(p, nr)) * r);
                  }
                  if (ok) {
                    fu.rule = FusedUpdate::LAMB;
                    fu.m = m, fu.v = v;
                    fu.beta1 = b1->name, fu.beta2 = b2->name;
                    fu.lr = lr ? lr->name : "", fu.decay = wd ? wd->name : "";
                    note_scale(gf);
                    return fu;
                  }
                }
            }
          }
        }
    }
  return fu;
}

// ---------------------------------------------------------------------------
// Schedule transformations.  Nodes are rewired IN PLACE, so the Stage handles
// the program holds stay valid.  (Reference: src/pipeline.cpp:851-902 split,
// 661-843 reorder, 471-587 asSlice.)
// ---------------------------------------------------------------------------
std::pair<Stage, Stage> Pipeline::split(Stage allReduce, SplitType type) {
  NodeRef ar = allReduce.node();
  if (type != AllReduceRSAG) fail("split: only AllReduceRSAG is implemented");
  if (!ar || ar->kind != NodeKind::AllReduce) fail("split: not an AllReduce stage");
  if (std::find(stages_.begin(), stages_.end(), ar) == stages_.end())
    fail("split: stage " + ar->name + " is not part of pipeline '" + name_ + "'");
  NodeRef rs = detail::makeStage(NodeKind::ReduceScatter, {ar->in[0]}, ar->type, Sliced);
  rs->red = ar->red;
  ar->kind = NodeKind::AllGather;  // same node, same handle: now gathers the scattered sum
  ar->in = {rs};
  ar->layout = Replicated;
  rediscover();
  return {Stage(Expression(rs)), Stage(Expression(ar))};
}

namespace {

// Replace every use of `from` inside the expression owned by stage `s`.
void substitute(const NodeRef &n, const NodeRef &from, const NodeRef &to, bool root) {
  if (!root && n->stage_id >= 0) return;
  for (NodeRef &c : n->in) {
    if (c.get() == from.get()) c = to;
    else substitute(c, from, to, false);
  }
  detail::relayout(*n);
}

}  // namespace

ReorderedStages Pipeline::reorder(std::vector<Stage> comps, Stage allGather) {
  NodeRef ag = allGather.node();
  if (!ag || ag->kind != NodeKind::AllGather) fail("reorder: the second argument must be an AllGather stage");
  const NodeRef sliced = ag->in[0];
  ReorderedStages out;
  std::set<const Node *> members;
  for (const Stage &c : comps) members.insert(c.node().get());
  // every consumer of the AllGather must move below it, or it would still need the gathered value
  for (const NodeRef &s : stages_) {
    if (members.count(s.get()) || s.get() == ag.get()) continue;
    std::vector<const Node *> d;
    direct_deps(s, true, &d);
    if (std::find(d.begin(), d.end(), ag.get()) != d.end())
      fail("reorder: stage " + s->name + " also uses the AllGather but is not among the reordered stages");
  }
  // What the moved stages read instead: the scattered value for the gathered
  // one, and, for an Update that now gathers, the slice it computed (on the
  // slice both hold the same numbers).
  std::vector<std::pair<NodeRef, NodeRef>> subs = {{ag, sliced}};
  // in topological order, so that a stage sees its producers already sliced
  for (const NodeRef &s : std::vector<NodeRef>(stages_)) {
    if (!members.count(s.get())) continue;
    std::vector<NodeRef> own;
    ownedNodes(s, true, &own);
    // Pointwise stages move; so does a Norm, which means the norm of the whole
    // (distributed) tensor whether its operand is gathered or still in slices.
    for (const NodeRef &n : own)
      if (isCollective(n->kind)) fail("reorder: stage " + s->name + " contains a collective");
    for (const auto &sub : subs) substitute(s, sub.first, sub.second, true);
    if (s->kind == NodeKind::Update && s->in[0]->layout == Replicated && s->in[1]->layout == Sliced) {
      // Update(w, f(gathered)) -> c = f(slice); Update(w, AllGather(c))
      NodeRef comp = s->in[1];
      if (comp->stage_id < 0) {  // an unnamed expression: give the sliced computation a stage of its own
        NodeRef named = detail::makeStage(comp->kind, comp->in, comp->type, comp->layout);
        named->op = comp->op, named->value = comp->value, named->scalar = comp->scalar;
        named->red = comp->red;
        comp = named;
      }
      NodeRef gather = std::make_shared<Node>();
      gather->kind = NodeKind::AllGather;
      gather->in = {comp};
      gather->type = comp->type;
      gather->layout = Replicated;
      s->in[1] = gather;
      s->layout = Replicated;
      subs.push_back({s, comp});
      out.compStages.push_back(Stage(Expression(comp)));
      out.allGatherStages.push_back(Stage(Expression(s)));
      // Later stages now read the slice computation, not this Update: it stays
      // part of the pipeline for its effect on the tensor.
      if (std::find(outputs_.begin(), outputs_.end(), s) == outputs_.end()) outputs_.push_back(s);
    } else {
      out.compStages.push_back(Stage(Expression(s)));
    }
  }
  rediscover();
  return out;
}

void Pipeline::asSlice(Tensor replicated) { asSlice(std::vector<Tensor>{replicated}); }

void Pipeline::asSlice(std::vector<Tensor> tensors) {
  for (const Tensor &t : tensors) {
    NodeRef tn = t.node();
    if (tn->kind != NodeKind::Tensor || tn->layout != Replicated)
      fail("asSlice: '" + tn->name + "' is not a Replicated tensor");
    // every use must already be on slices: a stage that needs the whole tensor forbids it
    for (const NodeRef &s : stages_) {
      std::vector<NodeRef> own;
      ownedNodes(s, true, &own);
      for (const NodeRef &n : own) {
        bool uses = false;
        for (const NodeRef &c : n->in) uses = uses || c.get() == tn.get();
        if (!uses) continue;
        if (n->kind == NodeKind::Update && n->in[0].get() == tn.get()) continue;  // handled below
        if (n->kind == NodeKind::Norm || isCollective(n->kind))
          fail("asSlice: '" + tn->name + "' is used whole by stage " + s->name);
        // a Replicated sub-expression inside a stage that works on the slice is
        // only ever evaluated at the slice's elements: the stage's layout decides
        if (s->layout != Sliced && !(n->kind == NodeKind::Scatter))
          fail("asSlice: stage " + s->name + " still computes on all of '" + tn->name +
               "'; reorder it below the AllGather first");
      }
    }
    tn->layout = Sliced;
    for (const NodeRef &s : stages_) {
      std::vector<NodeRef> own;
      ownedNodes(s, true, &own);
      for (const NodeRef &n : own) {
        if (n->kind == NodeKind::Update && n->in[0].get() == tn.get()) {
          if (n->in[1]->kind == NodeKind::AllGather) n->in[1] = n->in[1]->in[0];  // no gather needed
          n->layout = Sliced;
        } else if (n->kind == NodeKind::Scatter && n->in[0].get() == tn.get()) {
          // Scatter of a tensor that is already Sliced is the tensor itself
          n->kind = NodeKind::Cast;
          n->type = tn->type;
          n->layout = Sliced;
        } else {
          detail::relayout(*n);
          if (n->kind == NodeKind::Update && n->in[0]->layout == Replicated && n->in[1]->layout == Sliced &&
              n->in[1]->kind != NodeKind::AllGather)
            fail("asSlice: stage " + s->name + " would update Replicated '" + n->in[0]->name +
                 "' from a slice without an AllGather; reorder it below the AllGather first");
        }
      }
    }
  }
  rediscover();
}

void Autotuner::autotune(Pipeline &p, std::vector<Tensor> canSlice) {
  auto as_stages = [](const std::vector<NodeRef> &v) {
    std::vector<Stage> out;
    for (const NodeRef &n : v) out.push_back(Stage(Expression(n)));
    return out;
  };
  auto emit = [&](const std::string &schedule) {
    const std::string file = dir_ + "/" + p.name() + "-" + schedule + ".cu";
    p.codegen(file);
    emitted_.push_back(file);
  };
  // ---- AR_C: as written; every computation stage in one fusion group -----------
  NodeRef ar;
  std::vector<NodeRef> comps;
  for (const NodeRef &s : p.stages()) {
    if (s->kind == NodeKind::AllReduce) {
      if (ar) fail("autotune: pipeline '" + p.name() + "' has more than one AllReduce");
      ar = s;
    } else if (isCollective(s->kind)) {
      fail("autotune: write the pipeline with AllReduce only; the other schedules are derived");
    } else {
      comps.push_back(s);
    }
  }
  if (!ar) fail("autotune: pipeline '" + p.name() + "' has no AllReduce stage");
  if (comps.size() > 1) p.fuse(as_stages(comps));
  emit("AR_C");
  p.unfuse();  // the groups of this schedule do not carry over: the stages change

  // ---- RS_C_AG: split, move every consumer below the AllGather, slice the state --
  std::pair<Stage, Stage> rsag = p.split(Stage(Expression(ar)), AllReduceRSAG);
  std::vector<Stage> consumers;  // stages that depend on the gathered sum, directly or not
  {
    std::set<const Node *> dep = {rsag.second.node().get()};
    for (const NodeRef &s : p.stages()) {
      if (dep.count(s.get())) continue;
      std::vector<const Node *> d;
      direct_deps(s, true, &d);
      for (const Node *x : d)
        if (dep.count(x)) {
          dep.insert(s.get());
          consumers.push_back(Stage(Expression(s)));
          break;
        }
    }
  }
  ReorderedStages re = p.reorder(consumers, rsag.second);
  if (!canSlice.empty()) p.asSlice(canSlice);
  std::set<const Node *> gathers;
  for (const Stage &s : re.allGatherStages)
    if (s.node()->in[1]->kind == NodeKind::AllGather) gathers.insert(s.node().get());  // not sliced away
  std::vector<NodeRef> kernel;
  for (const NodeRef &s : p.stages())
    if (!isCollective(s->kind) && !gathers.count(s.get())) kernel.push_back(s);
  if (kernel.size() > 1) p.fuse(as_stages(kernel));
  emit("RS_C_AG");

  // ---- fuse_RS_C_AG: one kernel ----------------------------------------------------
  std::vector<NodeRef> all = p.stages();
  std::string why;
  if (!p.canFuse(all, &why)) {
    std::cerr << "coconet dsl: autotune: the fused schedule of '" << p.name()
              << "' is not emitted: " << why << std::endl;
    return;
  }
  bool has_norm = false;
  for (const NodeRef &s : all) has_norm = has_norm || s->kind == NodeKind::Norm;
  if (has_norm && p.classify(all).rule == FusedUpdate::Unknown) {
    // a global norm inside one kernel needs the two-phase kernel, which exists for LAMB only
    std::cerr << "coconet dsl: autotune: the fused schedule of '" << p.name()
              << "' is not emitted: it contains a Norm and is not LAMB" << std::endl;
    return;
  }
  p.fuse(as_stages(all));
  emit("fuse_RS_C_AG");
}

void Pipeline::print(std::ostream &os) const {
  os << "pipeline " << name_ << " {\n";
  for (const auto &g : groups()) {
    os << "  group:";
    for (const NodeRef &s : g) os << " " << s->name;
    os << "\n";
  }
  os << "}\n";
}

void Pipeline::codegen(const std::string &filename) {
  std::ofstream f(filename);
  if (!f) fail("cannot write " + filename);
  codegen(f);
}

}  // namespace ACCCDSL
