// Construction of the expression DAG and its layout / type rules.
#include "dsl.hpp"

#include <cstdio>
#include <cstdlib>

namespace ACCCDSL {

namespace {

int g_next_stage = 0;

[[noreturn]] void fail(const std::string &msg) {
  std::fprintf(stderr, "coconet dsl: %s\n", msg.c_str());
  std::exit(1);
}

NodeRef make(NodeKind k) {
  auto n = std::make_shared<Node>();
  n->kind = k;
  return n;
}

TensorElemType wider(TensorElemType a, TensorElemType b) {
  auto rank = [](TensorElemType t) {
    switch (t) {
      case Float64: return 6;
      case Float32: return 5;
      case Float16: return 4;
      case Int64: case UInt64: return 3;
      case Int32: case UInt32: return 2;
      default: return 1;
    }
  };
  return rank(a) >= rank(b) ? a : b;
}

// Layout of a pointwise result.  Scalars adopt the other operand's layout;
// Sliced wins over Replicated (the operation then runs on the slice only);
// Local values may only meet scalars or other Local values.
TensorLayout combine(const Node &a, const Node &b) {
  if (a.scalar) return b.layout;
  if (b.scalar) return a.layout;
  if (a.layout == b.layout) return a.layout;
  if (a.layout == Local || b.layout == Local)
    fail("a Local tensor ('" + (a.layout == Local ? a.name : b.name) +
         "') can only be combined with scalars or Local tensors; reduce it first");
  if ((a.layout == Sliced && b.layout == Replicated) || (a.layout == Replicated && b.layout == Sliced))
    return Sliced;
  fail("incompatible layouts in a pointwise operation");
}

NodeRef constant(double v, TensorElemType t) {
  NodeRef n = make(NodeKind::Const);
  n->value = v;
  n->type = t;
  n->scalar = true;
  return n;
}

Expression binary(char op, const NodeRef &a, const NodeRef &b) {
  if (!a || !b) fail("use of an uninitialised DSL object");
  NodeRef n = make(NodeKind::Binary);
  n->op = op;
  n->in = {a, b};
  // constants take the type of the other operand (1.0 - beta1 stays float)
  if (a->kind == NodeKind::Const) n->type = b->type;
  else if (b->kind == NodeKind::Const) n->type = a->type;
  else n->type = wider(a->type, b->type);
  n->scalar = a->scalar && b->scalar;
  n->layout = combine(*a, *b);
  return Expression(n);
}

}  // namespace

const char *elemTypeName(TensorElemType t) {
  switch (t) {
    case Float16: return "half";
    case Float32: return "float";
    case Float64: return "double";
    case Int8: return "char";
    case Int16: return "short";
    case Int32: return "int";
    case Int64: return "long";
    case UInt8: return "unsigned char";
    case UInt16: return "unsigned short";
    case UInt32: return "unsigned int";
    case UInt64: return "unsigned long";
    default: return "void";
  }
}

size_t elemTypeSize(TensorElemType t) {
  switch (t) {
    case Float16: case Int16: case UInt16: return 2;
    case Float32: case Int32: case UInt32: return 4;
    case Float64: case Int64: case UInt64: return 8;
    case Int8: case UInt8: return 1;
    default: return 0;
  }
}

bool isCollective(NodeKind k) {
  return k == NodeKind::AllReduce || k == NodeKind::ReduceScatter || k == NodeKind::AllGather ||
         k == NodeKind::Broadcast;
}

Variable::Variable(TensorElemType type, const std::string &name) {
  n_ = make(NodeKind::Variable);
  n_->type = type;
  n_->name = name;
  n_->scalar = true;
}

Tensor::Tensor(TensorElemType type, const Variable &size, TensorLayout layout,
               const std::string &name) {
  n_ = make(NodeKind::Tensor);
  n_->type = type;
  n_->name = name;
  n_->layout = layout;
  n_->dim = size.node();
}

Stage::Stage(const Expression &e) : Expression(e.node()) {
  if (!n_) fail("Stage built from an empty expression");
  if (n_->kind == NodeKind::Variable || n_->kind == NodeKind::Tensor || n_->kind == NodeKind::Const) {
    // `Stage x = w;` names a copy: keep inputs distinct from stages
    NodeRef src = n_;
    n_ = make(NodeKind::Binary);
    n_->op = '+';
    n_->in = {src, constant(0.0, src->type)};
    n_->type = src->type;
    n_->layout = src->layout;
    n_->scalar = src->scalar;
  }
  if (n_->stage_id < 0) {
    n_->stage_id = g_next_stage++;
    n_->name = "S" + std::to_string(n_->stage_id);
  }
}

Expression operator+(const Expression &a, const Expression &b) { return binary('+', a.node(), b.node()); }
Expression operator-(const Expression &a, const Expression &b) { return binary('-', a.node(), b.node()); }
Expression operator*(const Expression &a, const Expression &b) { return binary('*', a.node(), b.node()); }
Expression operator/(const Expression &a, const Expression &b) { return binary('/', a.node(), b.node()); }
Expression operator+(double a, const Expression &b) { return binary('+', constant(a, b.elemType()), b.node()); }
Expression operator-(double a, const Expression &b) { return binary('-', constant(a, b.elemType()), b.node()); }
Expression operator*(double a, const Expression &b) { return binary('*', constant(a, b.elemType()), b.node()); }
Expression operator/(double a, const Expression &b) { return binary('/', constant(a, b.elemType()), b.node()); }
Expression operator+(const Expression &a, double b) { return binary('+', a.node(), constant(b, a.elemType())); }
Expression operator-(const Expression &a, double b) { return binary('-', a.node(), constant(b, a.elemType())); }
Expression operator*(const Expression &a, double b) { return binary('*', a.node(), constant(b, a.elemType())); }
Expression operator/(const Expression &a, double b) { return binary('/', a.node(), constant(b, a.elemType())); }

Expression Const(TensorElemType type, double v) { return Expression(constant(v, type)); }

Expression Sqrt(const Expression &x) {
  NodeRef n = make(NodeKind::Sqrt);
  n->in = {x.node()};
  n->type = x.node()->type;
  n->layout = x.node()->layout;
  n->scalar = x.node()->scalar;
  return Expression(n);
}

Expression Norm(const Expression &x) {
  if (x.node()->layout == Local) fail("Norm of a Local tensor: reduce it first");
  NodeRef n = make(NodeKind::Norm);
  n->in = {x.node()};
  n->type = x.node()->type;
  n->layout = Replicated;
  n->scalar = true;
  return Expression(n);
}

Expression Cast(TensorElemType to, const Expression &x) {
  NodeRef n = make(NodeKind::Cast);
  n->in = {x.node()};
  n->type = to;
  n->layout = x.node()->layout;
  n->scalar = x.node()->scalar;
  return Expression(n);
}

Expression Scatter(const Expression &x) {
  if (x.node()->layout != Replicated) fail("Scatter needs a Replicated tensor ('" + x.name() + "')");
  NodeRef n = make(NodeKind::Scatter);
  n->in = {x.node()};
  n->type = x.node()->type;
  n->layout = Sliced;
  return Expression(n);
}

Expression AllReduce(ReduceOperation op, const Expression &x) {
  if (x.node()->layout != Local) fail("AllReduce needs a Local tensor ('" + x.name() + "')");
  NodeRef n = make(NodeKind::AllReduce);
  n->red = op;
  n->in = {x.node()};
  n->type = x.node()->type;
  n->layout = Replicated;
  return Expression(n);
}

Expression ReduceScatter(ReduceOperation op, const Expression &x) {
  if (x.node()->layout != Local) fail("ReduceScatter needs a Local tensor ('" + x.name() + "')");
  NodeRef n = make(NodeKind::ReduceScatter);
  n->red = op;
  n->in = {x.node()};
  n->type = x.node()->type;
  n->layout = Sliced;
  return Expression(n);
}

Expression AllGather(const Expression &x) {
  if (x.node()->layout != Sliced) fail("AllGather needs a Sliced value");
  NodeRef n = make(NodeKind::AllGather);
  n->in = {x.node()};
  n->type = x.node()->type;
  n->layout = Replicated;
  return Expression(n);
}

Expression Broadcast(const Expression &x, int root) {
  NodeRef n = make(NodeKind::Broadcast);
  n->in = {x.node()};
  n->value = root;
  n->type = x.node()->type;
  n->layout = Replicated;
  return Expression(n);
}

Expression Update(const Tensor &target, const Expression &value) {
  const Node &t = *target.node();
  NodeRef v = value.node();
  if (t.layout == Local) fail("Update of a Local tensor ('" + t.name + "')");
  if (v->layout == Local) fail("Update('" + t.name + "') from a Local value: reduce it first");
  if (t.layout == Replicated && v->layout == Sliced) v = AllGather(Expression(v)).node();  // implicit
  if (t.layout == Sliced && v->layout == Replicated && !v->scalar) v = Scatter(Expression(v)).node();
  NodeRef n = make(NodeKind::Update);
  n->in = {target.node(), v};
  n->type = t.type;
  n->layout = t.layout;
  return Expression(n);
}

namespace detail {

void relayout(Node &n) {
  switch (n.kind) {
    case NodeKind::Binary:
      n.scalar = n.in[0]->scalar && n.in[1]->scalar;
      n.layout = combine(*n.in[0], *n.in[1]);
      break;
    case NodeKind::Sqrt:
    case NodeKind::Cast:
      n.scalar = n.in[0]->scalar;
      n.layout = n.in[0]->layout;
      break;
    case NodeKind::Update:
      n.layout = n.in[0]->layout;
      break;
    default:
      break;
  }
}

NodeRef makeStage(NodeKind kind, const std::vector<NodeRef> &in, TensorElemType type,
                  TensorLayout layout) {
  NodeRef n = make(kind);
  n->in = in;
  n->type = type;
  n->layout = layout;
  n->stage_id = g_next_stage++;
  n->name = "S" + std::to_string(n->stage_id);
  return n;
}

}  // namespace detail

}  // namespace ACCCDSL
