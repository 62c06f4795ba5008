// Front-half IR of the i language as the B200 runtime sees it: parsed
// expressions, the component tree, canonical nodes and the wired graph.
//
// Mirrors the reference's data model so the recogniser can match on the same
// structure the reference compiler lowers:
//   Expr / PermutationAtom   compiler/src/ir/expr.rs:19-57
//   Component                compiler/src/ir/component.rs:17-41
//   Node / Site / AxisRef    compiler/src/ir/node.rs:25-68
//   Graph / Source           compiler/src/ir/graph.rs:20-60
#pragma once

#include <cstddef>
#include <memory>
#include <optional>
#include <string>
#include <utility>
#include <vector>

namespace ib {

enum class Op {
  Add, Mul, Div, Sub, Max, Min, Pow, Log,
  Gt, Ge, Lt, Le, Eq, Ne, And, Or, Xor, Not
};

const char* op_name(Op op);    // Rust Debug spelling: "Add", "Mul", ...
const char* op_token(Op op);   // source spelling: "+", "*", ...

struct PermAtom {
  enum Kind { Axis, Input, Bang } kind = Axis;
  char axis = 0;        // Axis
  size_t part = 0;      // Axis: number of apostrophes
  size_t input = 0;     // Input: operand 0 or 1
};

struct Expr {
  Op op = Op::Add;
  std::vector<std::string> inputs;   // index patterns, source order ("" = scalar)
  std::string output;
  std::vector<std::pair<char, std::vector<size_t>>> splits;
  std::vector<PermAtom> permutation;
  std::string source;                // original text, for plan dumps
};

struct Component;
using ComponentPtr = std::shared_ptr<const Component>;

struct Component {
  enum Kind { Identity, Leaf, Compose, Chain, Fanout, Pair, Swap } kind = Identity;
  Expr expr;              // Leaf
  ComponentPtr left;      // binary combinators; Swap uses left only
  ComponentPtr right;
};

struct AxisRef {
  size_t index = 0;
  size_t level = 0;
  bool operator==(const AxisRef& o) const { return index == o.index && level == o.level; }
};

struct Site {
  bool root = true;
  AxisRef at;
};

struct Node {
  Op op = Op::Add;
  size_t rank = 0;                               // number of canonical indexes
  std::vector<std::vector<size_t>> inputs;       // one multi-index per operand
  std::vector<size_t> output;
  std::vector<std::vector<size_t>> splits;       // per index, split factors
  std::vector<AxisRef> order;                    // loop levels, outer to inner
  std::vector<std::optional<Site>> compute_sites;
  std::optional<Site> init_site;
  std::string source;
  bool is_reduction() const { return output.size() < rank; }
};

struct Source {
  bool is_input = true;
  size_t index = 0;       // graph input number, or node number
  bool operator==(const Source& o) const { return is_input == o.is_input && index == o.index; }
};

struct GraphNode {
  Node inner;
  std::vector<Source> inputs;
};

struct Graph {
  size_t n_inputs = 0;
  std::vector<GraphNode> nodes;
  std::vector<Source> outputs;
};

// Error carried across the front half.  `text` is already in the form the C
// API reports (the reference reports Rust Debug renderings: core/src/lib.rs:69,
// 383-391).
struct Error {
  std::string text;
};

template <typename T>
struct Result {
  std::optional<T> value;
  Error error;
  bool ok() const { return value.has_value(); }
  static Result success(T v) { Result r; r.value = std::move(v); return r; }
  static Result failure(std::string text) { Result r; r.error.text = std::move(text); return r; }
};

// front/parser: text -> Expr
Result<Expr> parse_expr(const std::string& src);
// check/component: user-facing acceptance rules, "expr N: message"
std::optional<std::string> validate_component(const Component& c);
// lower: Expr -> Node, Component -> Graph
Result<Node> lower_expr_to_node(const Expr& e);
Result<Graph> lower_component_to_graph(const Component& c);

}  // namespace ib
