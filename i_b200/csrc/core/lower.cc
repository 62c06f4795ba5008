// Expr -> canonical Node, and Component tree -> wired Graph.
//
// Canonical index numbering: output axes first, then input axes in first-seen
// order (reference: compiler/src/lower/expr_to_node.rs:58-76).  With no
// permutation the loop order is index-major, level-minor (:116-127).  A staging
// digit or `!` attaches to the last axis part written before it, or to the root
// if none (:160-169).  The default init site of a reduction is the last output
// loop level of the order (compiler/src/check/node.rs:116-162); an explicit `!`
// may only sit at or inside it (:164-201).
//
// Wiring (compiler/src/lower/component_to_graph.rs): pair concatenates (:74-90);
// chain pairs p = min(|L.out|, |R.in|), inputs L.in ++ R.in[p..], outputs
// L.out[p..] ++ R.out (:92-116); compose(f, g) runs g first, inputs
// g.in ++ f.in[p..], outputs f.out ++ g.out[p..] (:118-141); fanout shares the
// first p = min(|L.in|, |R.in|) inputs (:143-163); swap exchanges outputs 0 and
// 1 when there are two (:64-70); identity is one input wired to one output
// (:25-29).  Node order is left nodes then right nodes (executed first first).
#include "ir.h"

#include <algorithm>
#include <map>
#include <set>

namespace ib {
namespace {

std::string lower_error(const std::string& message) {
  std::string escaped;
  for (char ch : message) {
    if (ch == '"' || ch == '\\') escaped.push_back('\\');
    escaped.push_back(ch);
  }
  return "LowerError { message: \"" + escaped + "\" }";
}

std::string site_text(const Site& s) {
  if (s.root) return "Root";
  return "At(" + std::to_string(s.at.index) + std::string(s.at.level, '\'') + ")";
}

// Default init site, or nullopt for a pointwise node.  Sets *err on failure.
std::optional<Site> required_init_site(const Node& n, const std::vector<AxisRef>& order,
                                       std::string* err) {
  std::set<size_t> out_idx(n.output.begin(), n.output.end());
  if (out_idx.size() == n.rank) return std::nullopt;
  size_t out_levels = 0;
  for (size_t idx : n.output) out_levels += n.splits[idx].size() + 1;
  Site site;
  if (out_levels == 0) return site;  // reduction to a scalar initialises at the root
  size_t seen = 0;
  std::optional<size_t> last;
  for (size_t pos = 0; pos < order.size(); ++pos)
    if (out_idx.count(order[pos].index)) {
      last = pos;
      ++seen;
    }
  if (seen != out_levels) {
    *err = "order does not contain every output loop level";
    return std::nullopt;
  }
  site.root = false;
  site.at = order[*last];
  return site;
}

std::optional<std::string> check_init_site(const Node& n, const std::vector<AxisRef>& order,
                                           const Site& site) {
  std::set<size_t> out_idx(n.output.begin(), n.output.end());
  size_t min_depth = 0;
  for (size_t pos = 0; pos < order.size(); ++pos)
    if (out_idx.count(order[pos].index)) min_depth = pos + 1;
  size_t depth = 0;
  if (!site.root) {
    auto it = std::find(order.begin(), order.end(), site.at);
    if (it == order.end()) return std::string("init site is outside loop order");
    depth = static_cast<size_t>(it - order.begin()) + 1;
  }
  if (depth < min_depth) {
    Site need;
    if (min_depth > 0) {
      need.root = false;
      need.at = order[min_depth - 1];
    }
    return "init site must be at or inside " + site_text(need);
  }
  return std::nullopt;
}

Result<Node> lower_expr_unchecked(const Expr& e) {
  std::vector<char> axes;
  auto note = [&](char axis) {
    if (std::find(axes.begin(), axes.end(), axis) == axes.end()) axes.push_back(axis);
  };
  for (char axis : e.output) note(axis);
  for (const auto& pattern : e.inputs)
    for (char axis : pattern) note(axis);
  std::map<char, size_t> number;
  for (size_t i = 0; i < axes.size(); ++i) number[axes[i]] = i;

  Node n;
  n.op = e.op;
  n.rank = axes.size();
  n.source = e.source;
  for (const auto& pattern : e.inputs) {
    std::vector<size_t> mi;
    for (char axis : pattern) mi.push_back(number[axis]);
    n.inputs.push_back(std::move(mi));
  }
  for (char axis : e.output) n.output.push_back(number[axis]);
  n.splits.assign(n.rank, {});
  for (const auto& split : e.splits) {
    auto it = number.find(split.first);
    if (it != number.end()) n.splits[it->second] = split.second;
  }
  n.compute_sites.assign(n.inputs.size(), std::nullopt);

  std::string err;
  if (e.permutation.empty()) {
    for (size_t idx = 0; idx < n.rank; ++idx)
      for (size_t level = 0; level <= n.splits[idx].size(); ++level)
        n.order.push_back(AxisRef{idx, level});
    n.init_site = required_init_site(n, n.order, &err);
    if (!err.empty()) return Result<Node>::failure(lower_error(err));
    return Result<Node>::success(std::move(n));
  }

  std::optional<AxisRef> last;
  std::optional<Site> explicit_init;
  for (const auto& atom : e.permutation) {
    Site here;
    if (last) {
      here.root = false;
      here.at = *last;
    }
    if (atom.kind == PermAtom::Axis) {
      auto it = number.find(atom.axis);
      if (it == number.end())
        return Result<Node>::failure(
            lower_error(std::string("unknown local axis `") + atom.axis + "`"));
      last = AxisRef{it->second, atom.part};
      n.order.push_back(*last);
    } else if (atom.kind == PermAtom::Input) {
      if (atom.input >= n.inputs.size())
        return Result<Node>::failure(lower_error("permutation references nonexistent input " +
                                                 std::to_string(atom.input)));
      n.compute_sites[atom.input] = here;
    } else {
      explicit_init = here;
    }
  }
  std::optional<Site> required = required_init_site(n, n.order, &err);
  if (!err.empty()) return Result<Node>::failure(lower_error(err));
  if (!required && explicit_init)
    return Result<Node>::failure(
        lower_error("pointwise node cannot have an output init directive"));
  if (required && explicit_init) {
    if (auto bad = check_init_site(n, n.order, *explicit_init))
      return Result<Node>::failure(lower_error(*bad));
    n.init_site = explicit_init;
  } else {
    n.init_site = required;
  }
  return Result<Node>::success(std::move(n));
}

struct Partial {
  size_t inputs = 0;
  std::vector<GraphNode> nodes;
  std::vector<Source> outputs;
  std::string error;
};

std::vector<Source> fresh_inputs(size_t base, size_t count) {
  std::vector<Source> out;
  for (size_t i = 0; i < count; ++i) out.push_back(Source{true, base + i});
  return out;
}

Source rewire(const Source& s, const std::vector<Source>& input_map, size_t node_offset) {
  if (s.is_input) return input_map[s.index];
  return Source{false, s.index + node_offset};
}

// Appends `part`'s nodes to `into` with its inputs replaced by `input_map`, and
// returns its outputs in the combined numbering.
std::vector<Source> splice(Partial&& part, const std::vector<Source>& input_map,
                           std::vector<GraphNode>* into) {
  const size_t offset = into->size();
  for (auto& node : part.nodes) {
    for (auto& src : node.inputs) src = rewire(src, input_map, offset);
    into->push_back(std::move(node));
  }
  std::vector<Source> outs;
  for (const auto& src : part.outputs) outs.push_back(rewire(src, input_map, offset));
  return outs;
}

Partial build(const Component& c) {
  Partial out;
  switch (c.kind) {
    case Component::Identity:
      out.inputs = 1;
      out.outputs = {Source{true, 0}};
      return out;
    case Component::Leaf: {
      Result<Node> node = lower_expr_unchecked(c.expr);
      if (!node.ok()) {
        out.error = node.error.text;
        return out;
      }
      GraphNode g;
      g.inputs = fresh_inputs(0, c.expr.inputs.size());
      g.inner = std::move(*node.value);
      out.inputs = c.expr.inputs.size();
      out.nodes.push_back(std::move(g));
      out.outputs = {Source{false, 0}};
      return out;
    }
    case Component::Swap: {
      out = build(*c.left);
      if (out.error.empty() && out.outputs.size() >= 2) std::swap(out.outputs[0], out.outputs[1]);
      return out;
    }
    default:
      break;
  }

  Partial l = build(*c.left);
  if (!l.error.empty()) return l;
  Partial r = build(*c.right);
  if (!r.error.empty()) return r;
  const size_t l_in = l.inputs, r_in = r.inputs;

  if (c.kind == Component::Pair) {
    auto lo = splice(std::move(l), fresh_inputs(0, l_in), &out.nodes);
    auto ro = splice(std::move(r), fresh_inputs(l_in, r_in), &out.nodes);
    out.inputs = l_in + r_in;
    out.outputs = lo;
    out.outputs.insert(out.outputs.end(), ro.begin(), ro.end());
  } else if (c.kind == Component::Chain) {
    const size_t p = std::min(l.outputs.size(), r_in);
    auto lo = splice(std::move(l), fresh_inputs(0, l_in), &out.nodes);
    std::vector<Source> map(lo.begin(), lo.begin() + p);
    auto rest = fresh_inputs(l_in, r_in - p);
    map.insert(map.end(), rest.begin(), rest.end());
    auto ro = splice(std::move(r), map, &out.nodes);
    out.inputs = l_in + r_in - p;
    out.outputs.assign(lo.begin() + p, lo.end());
    out.outputs.insert(out.outputs.end(), ro.begin(), ro.end());
  } else if (c.kind == Component::Compose) {
    const size_t p = std::min(l_in, r.outputs.size());
    auto ro = splice(std::move(r), fresh_inputs(0, r_in), &out.nodes);
    std::vector<Source> map(ro.begin(), ro.begin() + p);
    auto rest = fresh_inputs(r_in, l_in - p);
    map.insert(map.end(), rest.begin(), rest.end());
    auto lo = splice(std::move(l), map, &out.nodes);
    out.inputs = r_in + l_in - p;
    out.outputs = lo;
    out.outputs.insert(out.outputs.end(), ro.begin() + p, ro.end());
  } else {  // Fanout
    const size_t p = std::min(l_in, r_in);
    auto lo = splice(std::move(l), fresh_inputs(0, l_in), &out.nodes);
    std::vector<Source> map = fresh_inputs(0, p);
    auto rest = fresh_inputs(l_in, r_in - p);
    map.insert(map.end(), rest.begin(), rest.end());
    auto ro = splice(std::move(r), map, &out.nodes);
    out.inputs = l_in + r_in - p;
    out.outputs = lo;
    out.outputs.insert(out.outputs.end(), ro.begin(), ro.end());
  }
  return out;
}

}  // namespace

Result<Node> lower_expr_to_node(const Expr& e) {
  Component leaf;
  leaf.kind = Component::Leaf;
  leaf.expr = e;
  if (auto bad = validate_component(leaf)) return Result<Node>::failure(lower_error(*bad));
  return lower_expr_unchecked(e);
}

Result<Graph> lower_component_to_graph(const Component& c) {
  if (auto bad = validate_component(c)) return Result<Graph>::failure(lower_error(*bad));
  Partial p = build(c);
  if (!p.error.empty()) return Result<Graph>::failure(p.error);
  Graph g;
  g.n_inputs = p.inputs;
  g.nodes = std::move(p.nodes);
  g.outputs = std::move(p.outputs);
  return Result<Graph>::success(std::move(g));
}

}  // namespace ib
