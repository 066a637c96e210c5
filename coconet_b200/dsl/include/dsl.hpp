// CoCoNet's embedded DSL surface, re-implemented from scratch for the B200
// runtime: Variable / Tensor with Local / Replicated / Sliced layouts,
// collective and pointwise stages.  Source-compatible with the data-parallel
// example programs of parasailteam/coconet (examples/sgd/sgd.cpp,
// examples/adam/adam.cpp, examples/lamb/lamb.cpp; the surface they use is
// declared in the reference's src/dsl.hpp:97-167, 243-283, 400-429 and
// src/ast.hpp:48-102).
//
// Design: every DSL object is a handle to an immutable node of one expression
// DAG.  A `Stage` marks a node as a named pipeline stage.  There is no visitor
// hierarchy; the pipeline and the emitter walk the DAG directly.
#pragma once

#include <initializer_list>
#include <memory>
#include <string>
#include <vector>

namespace ACCCDSL {

enum TensorElemType { None = 0, Float16, Float32, Float64, Int8, Int16, Int32, Int64, UInt8, UInt16, UInt32, UInt64 };
enum TensorLayout { Replicated = 0, Sliced, Sliced_2, Local };
enum ReduceOperation { Summation = 0, Difference, Multiplication, Division, Maximum };

enum class NodeKind {
  Const, Variable, Tensor, Binary, Sqrt, Norm, Cast, Scatter,
  AllReduce, ReduceScatter, AllGather, Broadcast, Update
};

struct Node;
using NodeRef = std::shared_ptr<Node>;

struct Node {
  NodeKind kind = NodeKind::Const;
  TensorElemType type = Float32;
  TensorLayout layout = Replicated;
  bool scalar = false;            // Variable / Const / Norm: one value, not N of them
  std::string name;               // user name (Variable, Tensor) or S<k> (stages)
  double value = 0.0;             // Const
  char op = 0;                    // Binary: + - * /
  ReduceOperation red = Summation;
  std::vector<NodeRef> in;        // operands; Update: in[0] = target tensor, in[1] = value
  NodeRef dim;                    // Tensor: the Variable holding its element count
  int stage_id = -1;              // >= 0 once wrapped in a Stage
};

const char *elemTypeName(TensorElemType t);   // "float", "half", ...
size_t elemTypeSize(TensorElemType t);
bool isCollective(NodeKind k);

// Common handle.  Copying copies the handle, never the node.
class Expression {
 public:
  Expression() = default;
  explicit Expression(NodeRef n) : n_(std::move(n)) {}
  const NodeRef &node() const { return n_; }
  const std::string &name() const { return n_->name; }
  TensorLayout layout() const { return n_->layout; }
  TensorElemType elemType() const { return n_->type; }

 protected:
  NodeRef n_;
};

class Variable : public Expression {
 public:
  Variable(TensorElemType type, const std::string &name);
};

class Tensor : public Expression {
 public:
  Tensor(TensorElemType type, const Variable &size, TensorLayout layout, const std::string &name);
};

// A value that the pipeline computes.  Constructing one from an expression
// gives that expression's root a stage name (S0, S1, ... in creation order).
class Stage : public Expression {
 public:
  Stage(const Expression &e);  // NOLINT: implicit on purpose (Stage x = a + b;)
};

// ---- pointwise ------------------------------------------------------------
Expression operator+(const Expression &a, const Expression &b);
Expression operator-(const Expression &a, const Expression &b);
Expression operator*(const Expression &a, const Expression &b);
Expression operator/(const Expression &a, const Expression &b);
Expression operator+(double a, const Expression &b);
Expression operator-(double a, const Expression &b);
Expression operator*(double a, const Expression &b);
Expression operator/(double a, const Expression &b);
Expression operator+(const Expression &a, double b);
Expression operator-(const Expression &a, double b);
Expression operator*(const Expression &a, double b);
Expression operator/(const Expression &a, double b);
Expression Sqrt(const Expression &x);
Expression Norm(const Expression &x);                       // L2 norm over the whole tensor
Expression Cast(TensorElemType to, const Expression &x);
Expression Scatter(const Expression &replicated);           // this rank's slice of a Replicated tensor
Expression Const(TensorElemType type, double v);

// ---- collectives and updates ------------------------------------------------
Expression AllReduce(ReduceOperation op, const Expression &local);
Expression ReduceScatter(ReduceOperation op, const Expression &local);
Expression AllGather(const Expression &sliced);
Expression Broadcast(const Expression &x, int root);
// In-place update of a tensor.  A Sliced value assigned to a Replicated
// tensor implies an AllGather (reference: src/ast.hpp:966-968).
Expression Update(const Tensor &target, const Expression &value);

namespace detail {
// Recomputes type-independent attributes (layout, scalar) of a node from its
// operands after a schedule transformation rewired them.
void relayout(Node &n);
// A fresh stage node (gets the next S<k> name).
NodeRef makeStage(NodeKind kind, const std::vector<NodeRef> &in, TensorElemType type,
                  TensorLayout layout);
}  // namespace detail

}  // namespace ACCCDSL
