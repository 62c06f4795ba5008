// User-facing acceptance rules for a component tree.
//
// Each leaf expression is numbered in left-to-right tree order and checked
// against the rules of the reference's compiler/src/check/component.rs:
//   output axes unique (:63-74); unary output is a subset of the input
//   (:104-114); only + * > < && || ^^ reduce (:407-412); binary operators are
//   pointwise (:148-156); splits name local axes, once (:171-225); a
//   permutation lists every axis part exactly once, operands at most once, and
//   `!` only on reductions after all output parts (:227-338).
// Messages use the reference's wording, prefixed "expr N: " (:438-442).
#include "ir.h"

#include <map>
#include <set>

namespace ib {
namespace {

using AxisSet = std::set<char>;
using PartSet = std::set<std::pair<char, size_t>>;

std::string ticks(size_t n) { return std::string(n, '\''); }

bool reducible(Op op) {
  return op == Op::Add || op == Op::Mul || op == Op::Max || op == Op::Min || op == Op::And ||
         op == Op::Or || op == Op::Xor;
}

PartSet all_parts(const AxisSet& axes, const std::map<char, size_t>& split_parts) {
  PartSet out;
  for (char axis : axes) {
    auto it = split_parts.find(axis);
    size_t max_part = it == split_parts.end() ? 0 : it->second;
    for (size_t p = 0; p <= max_part; ++p) out.insert({axis, p});
  }
  return out;
}

std::optional<std::string> check_expr(const Expr& e) {
  AxisSet in_axes, out_axes;
  for (const auto& pattern : e.inputs) in_axes.insert(pattern.begin(), pattern.end());
  {
    AxisSet seen;
    for (char axis : e.output)
      if (!seen.insert(axis).second)
        return std::string("output pattern repeats axis `") + axis + "`";
    out_axes = seen;
  }
  const bool is_reduction = in_axes != out_axes;

  if (e.inputs.size() == 1) {
    for (char axis : out_axes)
      if (!in_axes.count(axis))
        return std::string("output axis `") + axis + "` does not appear in the input";
    if (e.op == Op::Not && is_reduction)
      return std::string("operator `Not` is only valid in unary pointwise form");
    if (is_reduction && !reducible(e.op))
      return std::string("operator `") + op_name(e.op) + "` is not reducible";
  } else if (e.inputs.size() == 2) {
    if (e.op == Op::Not) return std::string("operator `Not` is only valid in unary pointwise form");
    if (is_reduction)
      return std::string("binary operator `") + op_name(e.op) +
             "` must be pointwise; output axes must match the union of input axes";
  } else {
    return std::string("operator `") + op_name(e.op) + "` expects one or two inputs, found " +
           std::to_string(e.inputs.size());
  }

  AxisSet local = in_axes;
  local.insert(out_axes.begin(), out_axes.end());

  std::map<char, size_t> split_parts;
  for (const auto& split : e.splits) {
    if (!local.count(split.first))
      return std::string("split references unknown local axis `") + split.first + "`";
    if (split_parts.count(split.first))
      return std::string("duplicate split entry for axis `") + split.first + "`";
    split_parts[split.first] = split.second.size();
  }

  if (e.permutation.empty()) return std::nullopt;

  const PartSet expected = all_parts(local, split_parts);
  const PartSet output_parts = all_parts(out_axes, split_parts);
  PartSet seen;
  bool seen_input[2] = {false, false};
  bool seen_bang = false;
  for (const auto& atom : e.permutation) {
    if (atom.kind == PermAtom::Axis) {
      if (!local.count(atom.axis))
        return std::string("permutation references unknown local axis `") + atom.axis + "`";
      auto it = split_parts.find(atom.axis);
      size_t max_part = it == split_parts.end() ? 0 : it->second;
      if (atom.part > max_part)
        return std::string("permutation references nonexistent split part `") + atom.axis +
               ticks(atom.part) + "`";
      if (!seen.insert({atom.axis, atom.part}).second)
        return std::string("permutation repeats axis part `") + atom.axis + ticks(atom.part) + "`";
    } else if (atom.kind == PermAtom::Input) {
      if (atom.input >= e.inputs.size())
        return "permutation references nonexistent input " + std::to_string(atom.input);
      if (seen_input[atom.input])
        return "duplicate compute directive for input " + std::to_string(atom.input);
      seen_input[atom.input] = true;
    } else {
      if (seen_bang) return std::string("duplicate output init directive");
      if (local == out_axes)
        return std::string("output init directive is only valid for reductions");
      seen_bang = true;
      for (const auto& part : output_parts)
        if (!seen.count(part))
          return std::string("output init cannot appear before output axis part `") + part.first +
                 ticks(part.second) + "`";
    }
  }
  if (seen.size() != expected.size())
    return "permutation must list each local axis part exactly once; expected " +
           std::to_string(expected.size()) + ", found " + std::to_string(seen.size());
  for (const auto& part : expected)
    if (!seen.count(part))
      return std::string("permutation is missing axis part `") + part.first + ticks(part.second) +
             "`";
  return std::nullopt;
}

std::optional<std::string> walk(const Component& c, size_t* next_expr) {
  switch (c.kind) {
    case Component::Identity:
      return std::nullopt;
    case Component::Leaf: {
      size_t index = (*next_expr)++;
      if (auto message = check_expr(c.expr))
        return "expr " + std::to_string(index) + ": " + *message;
      return std::nullopt;
    }
    case Component::Swap:
      return walk(*c.left, next_expr);
    default:
      if (auto err = walk(*c.left, next_expr)) return err;
      return walk(*c.right, next_expr);
  }
}

}  // namespace

std::optional<std::string> validate_component(const Component& c) {
  size_t next_expr = 0;
  return walk(c, &next_expr);
}

}  // namespace ib
