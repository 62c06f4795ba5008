// Schedule acceptance: which compute-at placements the reference's loop-nest planner accepts,
// restated as a check over the wired graph so that `i_compile` refuses what the reference
// refuses, with the reference's message.
//
// A consumer that stages a producer inside its loops ("compute site" At(axis)) makes the
// producer run under the consumer's loops up to that axis: the producer's axes that line up with
// those loops are pruned (compiler/src/lower/node_to_stage.rs:611-783).  Two things can go wrong:
//
//  * the axes do not line up: a producer index and the consumer index that reads it must be split
//    the same way ("producer index .. has .. axes but consumer index .. has .. axes",
//    "producer extent kind .. does not match consumer extent kind ..", node_to_stage.rs:720-745);
//  * a reduction whose reduced axis is pruned is consumed before it is complete (an "online"
//    reduction).  The reference supports that for `+` and `>` only, by carrying a correction
//    (divisor, or exponent shift) along the fused chain until an accumulating `+` stage absorbs
//    it; the correction has to meet a division (for `+`) or a subtraction and then an
//    exponentiation (for `>`) on the way, and a chain that reaches a kernel's root stage with a
//    correction still pending is an error (compiler/src/lower/stage_to_kernel_program.rs:
//    366-380, 1158-1200, 1573-1653; the case of its test :2410-2431).
//
// Simplifications against the reference: corrections that the reference hoists to an outer stage
// are followed along the same fused edges (same accept / reject decision; the reference's
// "hoisted to a non-accumulator stage" wording is reported as the root message), and the check
// that a correction's shape broadcasts to the accumulator's is not made.
#include <algorithm>
#include <map>
#include <set>
#include <sstream>

#include "plan.h"

namespace ib {
namespace {

struct ExtentKind {
  enum Tag { Semantic, Base, Split } tag = Semantic;
  std::vector<size_t> factors;   // Base
  size_t level = 0, factor = 0;  // Split
  bool operator==(const ExtentKind& o) const {
    return tag == o.tag && factors == o.factors && level == o.level && factor == o.factor;
  }
  bool operator!=(const ExtentKind& o) const { return !(*this == o); }
};

// Rust `{:?}` of ir::common::ExtentKind.
std::string debug(const ExtentKind& k) {
  std::ostringstream out;
  if (k.tag == ExtentKind::Semantic) return "Semantic";
  if (k.tag == ExtentKind::Base) {
    out << "Base([";
    for (size_t i = 0; i < k.factors.size(); ++i) out << (i ? ", " : "") << k.factors[i];
    out << "])";
    return out.str();
  }
  out << "Split { level: " << k.level << ", factor: " << k.factor << " }";
  return out.str();
}

// node_to_stage.rs:593-609
ExtentKind extent_kind(const Node& node, const AxisRef& a) {
  ExtentKind k;
  const std::vector<size_t>& factors = node.splits[a.index];
  if (factors.empty()) return k;
  if (a.level == 0) {
    k.tag = ExtentKind::Base;
    k.factors = factors;
  } else {
    k.tag = ExtentKind::Split;
    k.level = a.level;
    k.factor = factors[a.level - 1];
  }
  return k;
}

std::pair<size_t, size_t> extent_order(const ExtentKind& k) {
  return k.tag == ExtentKind::Split ? std::make_pair(size_t(1), k.level) : std::make_pair(size_t(0), size_t(0));
}

struct AxisOf {
  size_t axis;       // position in the node's loop order
  ExtentKind kind;
};

// The node's axes over one index, base extent first, then the split levels.
std::vector<AxisOf> axes_for_index(const Node& node, size_t index) {
  std::vector<AxisOf> out;
  for (size_t a = 0; a < node.order.size(); ++a)
    if (node.order[a].index == index) out.push_back({a, extent_kind(node, node.order[a])});
  std::stable_sort(out.begin(), out.end(), [](const AxisOf& x, const AxisOf& y) {
    return extent_order(x.kind) < extent_order(y.kind);
  });
  return out;
}

bool in_output(const Node& node, size_t index) {
  return std::find(node.output.begin(), node.output.end(), index) != node.output.end();
}

// An online reduction's correction on its way to an accumulator.
struct Correction {
  enum Kind { Divisor, ExpShift } kind;
  enum State { Pending, Shifted, Ready } state = Pending;
  size_t origin;     // node that produced it (corrections are listed once per origin)
};

struct Checker {
  const Graph& g;
  std::string error;
  std::map<size_t, std::vector<Correction>> emitted;   // per fused node, as first emitted

  explicit Checker(const Graph& graph) : g(graph) {}

  bool fail(const std::string& message) {
    if (error.empty()) error = message;
    return false;
  }

  // node_to_stage.rs:694-783: producer axis -> consumer axis.
  bool align(const Node& producer, const Node& consumer, size_t input,
             std::map<size_t, size_t>* alignment) {
    const std::vector<size_t>& seen = consumer.inputs[input];
    if (producer.output.size() != seen.size())
      return fail("producer output has " + std::to_string(producer.output.size()) +
                  " shape dimensions but consumer input " + std::to_string(input) + " has " +
                  std::to_string(seen.size()) + " shape dimensions");
    std::set<size_t> taken;
    for (size_t dim = 0; dim < seen.size(); ++dim) {
      const auto pa = axes_for_index(producer, producer.output[dim]);
      const auto ca = axes_for_index(consumer, seen[dim]);
      if (pa.size() != ca.size())
        return fail("producer index " + std::to_string(producer.output[dim]) + " has " +
                    std::to_string(pa.size()) + " axes but consumer index " +
                    std::to_string(seen[dim]) + " has " + std::to_string(ca.size()) + " axes");
      for (size_t i = 0; i < pa.size(); ++i) {
        if (pa[i].kind != ca[i].kind)
          return fail("producer extent kind " + debug(pa[i].kind) +
                      " does not match consumer extent kind " + debug(ca[i].kind));
        (*alignment)[pa[i].axis] = ca[i].axis;
        taken.insert(ca[i].axis);
      }
    }
    // The producer's reduced axes line up with consumer axes over the same index number and of
    // the same extent kind, when exactly one such axis is still free.
    std::vector<std::pair<AxisOf, size_t>> reduced;
    for (size_t a = 0; a < producer.order.size(); ++a)
      if (!in_output(producer, producer.order[a].index))
        reduced.push_back({{a, extent_kind(producer, producer.order[a])}, producer.order[a].index});
    std::stable_sort(reduced.begin(), reduced.end(), [](const auto& x, const auto& y) {
      return extent_order(x.first.kind) < extent_order(y.first.kind);
    });
    for (const auto& [axis, index] : reduced) {
      if (alignment->count(axis.axis)) continue;
      if (index >= consumer.rank) continue;
      std::vector<size_t> candidates;
      for (const AxisOf& c : axes_for_index(consumer, index))
        if (!taken.count(c.axis) && c.kind == axis.kind) candidates.push_back(c.axis);
      if (candidates.size() == 1) {
        (*alignment)[axis.axis] = candidates[0];
        taken.insert(candidates[0]);
      } else if (candidates.size() > 1) {
        return fail("producer reduced axis " + std::to_string(axis.axis) +
                    " ambiguously aligns with consumer index " + std::to_string(index));
      }
    }
    return true;
  }

  // stage_to_kernel_program.rs:1594-1637
  bool pass_through(const Node& stage, size_t input, Correction* c) {
    if (c->state == Correction::Ready) return true;
    if (c->kind == Correction::Divisor) {
      if (c->state == Correction::Pending && stage.op == Op::Div && input > 0) {
        c->state = Correction::Ready;
        return true;
      }
      if (c->state == Correction::Pending)
        return fail("online reduction correction requires a division use before accumulation");
      return fail("division correction reached invalid shifted state");
    }
    if (c->state == Correction::Pending) {
      if (stage.op == Op::Sub && input > 0) {
        c->state = Correction::Shifted;
        return true;
      }
      return fail("online max correction requires a subtraction use before exponentiation");
    }
    if (stage.op == Op::Pow) {
      c->state = Correction::Ready;
      return true;
    }
    return fail("online max correction requires exponentiation before accumulation");
  }

  // Corrections that leave `n`, computed under a consumer that prunes the axes in `pruned`
  // (empty for a kernel's root stage).
  bool emit(size_t n, const std::set<size_t>& pruned, bool is_root, std::vector<Correction>* out) {
    if (!is_root) {
      auto done = emitted.find(n);
      if (done != emitted.end()) {
        *out = done->second;
        return true;
      }
    }
    const Node& stage = g.nodes[n].inner;
    std::vector<Correction> outgoing;
    auto add_once = [&](const Correction& c) {
      for (const Correction& have : outgoing)
        if (have.origin == c.origin && have.kind == c.kind && have.state == c.state) return;
      outgoing.push_back(c);
    };
    for (size_t k = 0; k < stage.inputs.size(); ++k) {
      const Source& src = g.nodes[n].inputs[k];
      if (src.is_input) continue;
      std::vector<Correction> incoming;
      if (stage.compute_sites[k]) {
        const Node& producer = g.nodes[src.index].inner;
        std::map<size_t, size_t> alignment;
        if (!align(producer, stage, k, &alignment)) return false;
        // The consumer's loops down to the site (node_to_stage.rs:668-692).
        size_t prefix = 0;
        const Site& site = *stage.compute_sites[k];
        if (!site.root) {
          for (size_t a = 0; a < stage.order.size(); ++a)
            if (stage.order[a] == site.at) prefix = a + 1;
        }
        std::set<size_t> producer_pruned;
        for (const auto& [pa, ca] : alignment)
          if (ca < prefix) producer_pruned.insert(pa);
        if (!emit(src.index, producer_pruned, false, &incoming)) return false;
      } else {
        // Not staged here, but possibly emitted already under a sibling in the same kernel.
        auto done = emitted.find(src.index);
        if (done != emitted.end()) incoming = done->second;
      }
      if (incoming.empty()) continue;
      const bool all_ready = std::all_of(incoming.begin(), incoming.end(), [](const Correction& c) {
        return c.state == Correction::Ready;
      });
      if (stage.op == Op::Add && stage.is_reduction() && all_ready) continue;   // absorbed here
      if (stage.is_reduction()) {
        if (stage.op == Op::Add)
          return fail("online reduction correction reached accumulator before correction use");
        return fail("online reduction correction reached unsupported accumulator");
      }
      for (Correction c : incoming) {
        if (!pass_through(stage, k, &c)) return false;
        add_once(c);
      }
    }
    // This stage's own reduction is online when one of its reduced axes is driven by the consumer.
    if (!is_root && stage.is_reduction()) {
      bool online = false;
      for (size_t a : pruned)
        if (!in_output(stage, stage.order[a].index)) online = true;
      if (online) {
        if (stage.op == Op::Add) add_once(Correction{Correction::Divisor, Correction::Pending, n});
        else if (stage.op == Op::Max) add_once(Correction{Correction::ExpShift, Correction::Pending, n});
        else
          return fail("stage " + std::to_string(n) +
                      " requires online reduction lowering: fused reduction axis is consumed before completion");
      }
    }
    if (!is_root) emitted[n] = outgoing;
    *out = outgoing;
    return true;
  }
};

}  // namespace

// Returns the reference's message when the graph's compute-at placements are ones the
// reference's planner rejects; nothing otherwise.
std::optional<std::string> check_schedule(const Graph& g) {
  // A node is staged when a consumer reads it through a compute site; every other node is the
  // root stage of a kernel of its own.
  std::vector<bool> staged(g.nodes.size(), false);
  for (const GraphNode& node : g.nodes)
    for (size_t k = 0; k < node.inputs.size(); ++k)
      if (!node.inputs[k].is_input && node.inner.compute_sites[k]) staged[node.inputs[k].index] = true;
  for (size_t n = 0; n < g.nodes.size(); ++n) {
    if (staged[n]) continue;
    Checker checker(g);
    std::vector<Correction> left;
    if (!checker.emit(n, {}, true, &left)) return checker.error;
    if (!left.empty()) return std::string("online reduction correction reached root without an accumulator");
  }
  return std::nullopt;
}

}  // namespace ib
