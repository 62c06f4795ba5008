// Recogniser: Graph -> Plan.
//
// Pass 1 turns every node into a Map or Reduce step (scalar semantics of the
// reference's compiler/src/lower/exec_plan_to_module.rs:592-640).
// Pass 2 folds `Mul node -> Add-reduce node` pairs into Contract steps
// (the reference's `ik*jk~ijk >> +ijk~ij`, README.md:16).
// Pass 3 folds `max, sub, exp, sum, div` chains into RowSoftmax steps
// (README.md:19-25).
// Pass 4 folds Contract -> RowSoftmax -> Contract into one Attention step
// (README.md:31), the graph the reference emits as one kernel in
// ilang-python/annotated-flashattn.c:52-310.
#include "plan.h"

#include <algorithm>
#include <cstdlib>
#include <map>
#include <set>
#include <sstream>

namespace ib {
namespace {

std::string lower_error(const std::string& message) {
  return "LowerError { message: \"" + message + "\" }";
}

// I_B200_FUSE_ATTENTION=always fuses every recognised attention chain,
// whatever its schedule says.
bool fuse_always() {
  const char* env = std::getenv("I_B200_FUSE_ATTENTION");
  return env && std::string(env) == "always";
}

bool is_iota(const std::vector<size_t>& v, size_t n) {
  if (v.size() != n) return false;
  for (size_t i = 0; i < n; ++i)
    if (v[i] != i) return false;
  return true;
}

bool has_repeat(const std::vector<size_t>& v) {
  std::set<size_t> s(v.begin(), v.end());
  return s.size() != v.size();
}

struct Builder {
  const Graph& g;
  std::vector<bool> is_output;
  std::vector<Step> steps;           // indexed by owning node; kind valid if alive
  std::vector<bool> alive;

  explicit Builder(const Graph& graph) : g(graph) {
    is_output.assign(g.nodes.size(), false);
    for (const auto& src : g.outputs)
      if (!src.is_input) is_output[src.index] = true;
  }

  // Live steps that read node `n`, each listed once.
  std::vector<size_t> readers(size_t n) const {
    std::vector<size_t> out;
    for (size_t i = 0; i < g.nodes.size(); ++i) {
      if (!alive[i]) continue;
      bool reads = false;
      for (const auto& acc : steps[i].in) reads = reads || (!acc.buffer.is_input && acc.buffer.index == n);
      for (const auto& acc : steps[i].epilogue_in)
        reads = reads || (!acc.buffer.is_input && acc.buffer.index == n);
      if (reads) out.push_back(i);
    }
    return out;
  }

  // The only live step reading node `n`, provided `n` is not a graph output.
  std::optional<size_t> sole_reader(size_t n) const {
    if (is_output[n]) return std::nullopt;
    std::vector<size_t> r = readers(n);
    if (r.size() != 1) return std::nullopt;
    return r[0];
  }
};

std::optional<std::string> basic_steps(Builder& b) {
  const Graph& g = b.g;
  b.steps.resize(g.nodes.size());
  b.alive.assign(g.nodes.size(), true);
  for (size_t n = 0; n < g.nodes.size(); ++n) {
    const Node& node = g.nodes[n].inner;
    for (size_t i = 0; i < node.inputs.size(); ++i)
      if (g.nodes[n].inputs[i].is_input && node.compute_sites[i])
        return lower_error("node " + std::to_string(n) + " input " + std::to_string(i) +
                           " is a graph input with a compute site");
    Step& s = b.steps[n];
    s.kind = node.is_reduction() ? StepKind::Reduce : StepKind::Map;
    s.op = node.op;
    s.rank = node.rank;
    for (size_t i = 0; i < node.inputs.size(); ++i)
      s.in.push_back(Access{g.nodes[n].inputs[i], node.inputs[i]});
    s.out = Access{Source{false, n}, node.output};
    s.nodes = {n};
    // Staging at the root hoists the producer in front of the loops, which
    // materialises it; only a site inside the loops fuses.
    for (const auto& site : node.compute_sites)
      if (site && !site->root) s.hint.staged = true;
  }
  return std::nullopt;
}

// Classifies a fused Mul/Add-reduce pair as a batched GEMM, if it is one.
bool classify_contraction(const Step& mul, const std::vector<size_t>& out_idx, ContractForm* form) {
  const auto& a = mul.in[0].index;
  const auto& bb = mul.in[1].index;
  if (has_repeat(a) || has_repeat(bb) || has_repeat(out_idx)) return false;
  auto in = [](const std::vector<size_t>& v, size_t x) {
    return std::find(v.begin(), v.end(), x) != v.end();
  };
  std::vector<size_t> batch, ms, ns, ks;
  for (size_t x = 0; x < mul.rank; ++x) {
    bool i0 = in(a, x), i1 = in(bb, x), o = in(out_idx, x);
    if (i0 && i1 && o) batch.push_back(x);
    else if (i0 && !i1 && o) ms.push_back(x);
    else if (!i0 && i1 && o) ns.push_back(x);
    else if (i0 && i1 && !o) ks.push_back(x);
    else return false;
  }
  if (ks.size() != 1 || ms.size() > 1 || ns.size() > 1) return false;
  const size_t nb = batch.size();
  // Batch axes lead all three tensors in the same order.
  std::vector<size_t> lead(a.begin(), a.begin() + std::min(nb, a.size()));
  if (lead.size() != nb) return false;
  for (size_t x : lead)
    if (std::find(batch.begin(), batch.end(), x) == batch.end()) return false;
  if (bb.size() < nb || out_idx.size() < nb) return false;
  for (size_t i = 0; i < nb; ++i)
    if (bb[i] != lead[i] || out_idx[i] != lead[i]) return false;

  form->n_batch = nb;
  form->k = ks[0];
  form->has_m = !ms.empty();
  form->has_n = !ns.empty();
  form->m = form->has_m ? ms[0] : 0;
  form->n = form->has_n ? ns[0] : 0;
  // Operand 0: [.., m, k] or [.., k, m] (or [.., k] without m).
  std::vector<size_t> ta(a.begin() + nb, a.end());
  if (form->has_m) {
    if (ta == std::vector<size_t>{form->m, form->k}) form->a_kmajor = true;
    else if (ta == std::vector<size_t>{form->k, form->m}) form->a_kmajor = false;
    else return false;
  } else {
    if (ta != std::vector<size_t>{form->k}) return false;
    form->a_kmajor = true;
  }
  std::vector<size_t> tb(bb.begin() + nb, bb.end());
  if (form->has_n) {
    if (tb == std::vector<size_t>{form->n, form->k}) form->b_kmajor = true;
    else if (tb == std::vector<size_t>{form->k, form->n}) form->b_kmajor = false;
    else return false;
  } else {
    if (tb != std::vector<size_t>{form->k}) return false;
    form->b_kmajor = true;
  }
  std::vector<size_t> to(out_idx.begin() + nb, out_idx.end());
  std::vector<size_t> want;
  if (form->has_m) want.push_back(form->m);
  if (form->has_n) want.push_back(form->n);
  if (to == want) {
    form->swap_out = false;
  } else {
    std::reverse(want.begin(), want.end());
    if (to != want) return false;
    form->swap_out = true;
  }
  return true;
}

void fuse_contractions(Builder& b) {
  for (size_t n = 0; n < b.g.nodes.size(); ++n) {
    if (!b.alive[n]) continue;
    Step& mul = b.steps[n];
    if (mul.kind != StepKind::Map || mul.op != Op::Mul || mul.in.size() != 2) continue;
    auto reader = b.sole_reader(n);
    if (!reader) continue;
    Step& red = b.steps[*reader];
    if (red.kind != StepKind::Reduce || red.op != Op::Add || red.in.size() != 1) continue;
    const auto& view = red.in[0].index;           // reducer's index per dim of the product
    if (view.size() != mul.out.index.size() || has_repeat(view)) continue;
    std::map<size_t, size_t> to_mul;              // reducer index -> multiplier index
    for (size_t p = 0; p < view.size(); ++p) to_mul[view[p]] = mul.out.index[p];
    std::vector<size_t> out_idx;
    for (size_t x : red.out.index) out_idx.push_back(to_mul[x]);
    ContractForm form;
    if (!classify_contraction(mul, out_idx, &form)) continue;

    Step fused;
    fused.kind = StepKind::Contract;
    fused.op = Op::Add;
    fused.rank = mul.rank;
    fused.in = mul.in;
    fused.out = Access{red.out.buffer, out_idx};
    fused.form = form;
    fused.nodes = {n, *reader};
    fused.hint.staged = red.hint.staged;
    const Node& mnode = b.g.nodes[n].inner;
    if (form.has_m && !mnode.splits[form.m].empty()) fused.hint.row_split = mnode.splits[form.m][0];
    if (form.has_n && !mnode.splits[form.n].empty()) fused.hint.col_split = mnode.splits[form.n][0];
    for (const auto& level : mnode.order)
      if ((form.has_n && level.index == form.n) || (form.has_m && level.index == form.m)) {
        fused.hint.reduce_outer = form.has_n && level.index == form.n;
        break;
      }
    b.steps[*reader] = std::move(fused);
    b.alive[n] = false;
  }
}

// A reduce over exactly the last axis of its operand, leading axes kept in order.
bool is_row_reduce(const Step& s, Op op) {
  if (s.kind != StepKind::Reduce || s.op != op || s.in.size() != 1) return false;
  return s.rank >= 1 && is_iota(s.in[0].index, s.rank) && is_iota(s.out.index, s.rank - 1);
}

// x[.., r, c] (op) v[.., r] -> [.., r, c]
bool is_row_broadcast(const Step& s, Op op) {
  if (s.kind != StepKind::Map || s.op != op || s.in.size() != 2) return false;
  return s.rank >= 1 && is_iota(s.in[0].index, s.rank) && is_iota(s.in[1].index, s.rank - 1) &&
         is_iota(s.out.index, s.rank);
}

void fuse_softmax(Builder& b) {
  for (size_t n = 0; n < b.g.nodes.size(); ++n) {
    if (!b.alive[n] || !is_row_reduce(b.steps[n], Op::Max)) continue;
    const Step& mx = b.steps[n];
    auto r_sub = b.sole_reader(n);
    if (!r_sub || !is_row_broadcast(b.steps[*r_sub], Op::Sub)) continue;
    const Step& sub = b.steps[*r_sub];
    if (!(sub.in[0].buffer == mx.in[0].buffer) || sub.in[1].buffer.is_input ||
        sub.in[1].buffer.index != n)
      continue;
    auto r_exp = b.sole_reader(*r_sub);
    if (!r_exp) continue;
    const Step& ex = b.steps[*r_exp];
    if (ex.kind != StepKind::Map || ex.op != Op::Pow || ex.in.size() != 1 ||
        !is_iota(ex.in[0].index, ex.rank) || !is_iota(ex.out.index, ex.rank))
      continue;
    if (b.is_output[*r_exp]) continue;
    std::vector<size_t> rd = b.readers(*r_exp);
    if (rd.size() != 2) continue;
    size_t i_sum = rd[0], i_div = rd[1];
    if (!is_row_reduce(b.steps[i_sum], Op::Add)) std::swap(i_sum, i_div);
    if (!is_row_reduce(b.steps[i_sum], Op::Add) || !is_row_broadcast(b.steps[i_div], Op::Div))
      continue;
    const Step& dv = b.steps[i_div];
    if (dv.in[0].buffer.is_input || dv.in[0].buffer.index != *r_exp || dv.in[1].buffer.is_input ||
        dv.in[1].buffer.index != i_sum)
      continue;
    if (b.is_output[i_sum] || b.readers(i_sum).size() != 1) continue;

    Step fused;
    fused.kind = StepKind::RowSoftmax;
    fused.op = Op::Div;
    fused.rank = mx.rank;
    fused.in = {mx.in[0]};
    fused.out = dv.out;
    fused.nodes = {n, *r_sub, *r_exp, i_sum, i_div};
    const Node& mnode = b.g.nodes[n].inner;
    const size_t col = mx.rank - 1;
    if (mx.rank >= 2 && !mnode.splits[col - 1].empty()) fused.hint.row_split = mnode.splits[col - 1][0];
    if (!mnode.splits[col].empty()) fused.hint.col_split = mnode.splits[col][0];
    // Which of the row / reduced axes has the outermost loop (batch axes aside).
    for (const auto& level : mnode.order)
      if (level.index == col || (mx.rank >= 2 && level.index == col - 1)) {
        fused.hint.reduce_outer = level.index == col;
        break;
      }
    fused.hint.staged = b.steps[*r_sub].hint.staged || ex.hint.staged || dv.hint.staged;
    const size_t last = std::max(std::max(*r_sub, *r_exp), std::max(i_sum, i_div));
    for (size_t dead : fused.nodes) b.alive[dead] = false;
    fused.out.buffer = Source{false, i_div};
    // The fused step takes the slot of the last node of the group; its result
    // still belongs to the divide node.
    b.steps[last] = std::move(fused);
    b.alive[last] = true;
  }
}

void fuse_attention(Builder& b) {
  for (size_t n = 0; n < b.g.nodes.size(); ++n) {
    if (!b.alive[n] || b.steps[n].kind != StepKind::Contract) continue;
    const Step& qk = b.steps[n];
    const ContractForm& f1 = qk.form;
    if (!f1.has_m || !f1.has_n || !f1.a_kmajor || !f1.b_kmajor || f1.swap_out) continue;
    const size_t s_node = qk.out.buffer.index;
    auto r_sm = b.sole_reader(s_node);
    // Optionally one scalar on the logits between the contraction and the softmax
    // (`.*ik~ik`, `ik*.~ik`, `ik/.~ik`): carried as a fourth operand of the fused step.
    std::optional<size_t> scale_slot;
    Access scale_operand;
    bool scale_divides = false;
    if (r_sm && b.steps[*r_sm].kind == StepKind::Map && b.steps[*r_sm].in.size() == 2) {
      const Step& sc = b.steps[*r_sm];
      const bool s_first = !sc.in[0].buffer.is_input && sc.in[0].buffer.index == s_node;
      const Access& s_side = sc.in[s_first ? 0 : 1];
      const Access& c_side = sc.in[s_first ? 1 : 0];
      const bool shape_ok = sc.rank == qk.out.index.size() && is_iota(sc.out.index, sc.rank) &&
                            is_iota(s_side.index, sc.rank) && c_side.index.empty() &&
                            !s_side.buffer.is_input && s_side.buffer.index == s_node &&
                            !(!c_side.buffer.is_input && c_side.buffer.index == s_node);
      const bool op_ok = sc.op == Op::Mul || (sc.op == Op::Div && s_first);
      if (shape_ok && op_ok) {
        scale_slot = *r_sm;
        scale_operand = c_side;
        scale_divides = sc.op == Op::Div;
        r_sm = b.sole_reader(sc.out.buffer.index);
      }
    }
    if (!r_sm || b.steps[*r_sm].kind != StepKind::RowSoftmax) continue;
    const Step& sm = b.steps[*r_sm];
    if (sm.rank != f1.n_batch + 2) continue;
    const size_t p_node = sm.out.buffer.index;
    auto r_pv = b.sole_reader(p_node);
    if (!r_pv || b.steps[*r_pv].kind != StepKind::Contract) continue;
    const Step& pv = b.steps[*r_pv];
    const ContractForm& f2 = pv.form;
    if (pv.in[0].buffer.is_input || pv.in[0].buffer.index != p_node) continue;
    if (!f2.has_m || !f2.has_n || !f2.a_kmajor || f2.swap_out || f2.n_batch != f1.n_batch) continue;
    // The schedule decides fusion, as in the reference: the chain becomes one
    // kernel only when the second contraction stages its P operand inside its
    // loops (README.md:28, `ji0i'kj'`); the naive schedule of
    // ilang-python/flash-attn.py:57-65 keeps S and P as full intermediates.
    const Node& pv_mul = b.g.nodes[pv.nodes[0]].inner;
    const bool p_staged = pv_mul.compute_sites[0] && !pv_mul.compute_sites[0]->root;
    if (!p_staged && !fuse_always()) continue;

    Step fused;
    fused.kind = StepKind::Attention;
    fused.op = Op::Add;
    fused.rank = qk.rank;
    fused.in = {qk.in[0], qk.in[1], pv.in[1]};
    if (scale_slot) {
      fused.in.push_back(scale_operand);
      fused.op = scale_divides ? Op::Div : Op::Mul;     // how the fourth operand meets the logits
    }
    fused.out = pv.out;
    fused.form = f1;
    fused.form2 = f2;
    fused.hint = sm.hint;
    fused.hint.staged = pv.hint.staged || sm.hint.staged;
    fused.nodes = qk.nodes;
    if (scale_slot)
      fused.nodes.insert(fused.nodes.end(), b.steps[*scale_slot].nodes.begin(),
                         b.steps[*scale_slot].nodes.end());
    fused.nodes.insert(fused.nodes.end(), sm.nodes.begin(), sm.nodes.end());
    fused.nodes.insert(fused.nodes.end(), pv.nodes.begin(), pv.nodes.end());
    const size_t slot = *r_pv, sm_slot = *r_sm;
    b.alive[n] = false;
    if (scale_slot) b.alive[*scale_slot] = false;
    b.alive[sm_slot] = false;
    b.steps[slot] = std::move(fused);
  }
}

// Attention written with the normalisation deferred: E = exp(S) or exp(S - rowmax S),
// O = (E V) / rowsum E — `mm_t >> exp >> (mm & row_sum) >> row_div`, the form the reference's
// tests build in compiler/src/lower/stage_to_kernel_program.rs:2705-2780.  It is the same
// function of Q, K, V as the README chain wherever exp(S) is finite, and the fused kernel
// subtracts the running maximum in any case, so it also stays finite where the unshifted
// form would overflow.  The schedule gate is the one of fuse_attention.
void fuse_deferred_attention(Builder& b) {
  auto is_exp = [](const Step& s) {
    return s.kind == StepKind::Map && s.op == Op::Pow && s.in.size() == 1 &&
           is_iota(s.in[0].index, s.rank) && is_iota(s.out.index, s.rank);
  };
  auto reads = [](const Access& a, size_t node) { return !a.buffer.is_input && a.buffer.index == node; };
  for (size_t n = 0; n < b.g.nodes.size(); ++n) {
    if (!b.alive[n] || b.steps[n].kind != StepKind::Contract) continue;
    const Step& qk = b.steps[n];
    const ContractForm& f1 = qk.form;
    if (!f1.has_m || !f1.has_n || !f1.a_kmajor || !f1.b_kmajor || f1.swap_out) continue;
    const size_t s_node = qk.out.buffer.index;
    if (b.is_output[s_node]) continue;
    std::vector<size_t> group = qk.nodes;
    std::vector<size_t> slots = {n};
    // exp directly on S, or on S - rowmax S.
    std::vector<size_t> rd = b.readers(s_node);
    size_t i_exp;
    if (rd.size() == 1 && is_exp(b.steps[rd[0]])) {
      i_exp = rd[0];
    } else if (rd.size() == 2) {
      size_t i_max = rd[0], i_sub = rd[1];
      if (!is_row_reduce(b.steps[i_max], Op::Max)) std::swap(i_max, i_sub);
      const Step& mx = b.steps[i_max];
      const Step& sub = b.steps[i_sub];
      if (!is_row_reduce(mx, Op::Max) || !is_row_broadcast(sub, Op::Sub)) continue;
      const size_t m_node = mx.out.buffer.index;
      if (!reads(mx.in[0], s_node) || !reads(sub.in[0], s_node) || !reads(sub.in[1], m_node)) continue;
      if (b.is_output[m_node] || b.readers(m_node).size() != 1) continue;
      const size_t y_node = sub.out.buffer.index;
      auto r_exp = b.sole_reader(y_node);
      if (!r_exp || !is_exp(b.steps[*r_exp])) continue;
      i_exp = *r_exp;
      slots.push_back(i_max);
      slots.push_back(i_sub);
      group.insert(group.end(), mx.nodes.begin(), mx.nodes.end());
      group.insert(group.end(), sub.nodes.begin(), sub.nodes.end());
    } else {
      continue;
    }
    const Step& ex = b.steps[i_exp];
    if (ex.rank != f1.n_batch + 2) continue;
    const size_t e_node = ex.out.buffer.index;
    if (b.is_output[e_node]) continue;
    // E feeds the second contraction and the row sum.
    rd = b.readers(e_node);
    if (rd.size() != 2) continue;
    size_t i_pv = rd[0], i_sum = rd[1];
    if (b.steps[i_pv].kind != StepKind::Contract) std::swap(i_pv, i_sum);
    const Step& pv = b.steps[i_pv];
    const Step& sum = b.steps[i_sum];
    if (pv.kind != StepKind::Contract || !is_row_reduce(sum, Op::Add)) continue;
    if (!reads(pv.in[0], e_node) || !reads(sum.in[0], e_node)) continue;
    const ContractForm& f2 = pv.form;
    if (!f2.has_m || !f2.has_n || !f2.a_kmajor || f2.swap_out || f2.n_batch != f1.n_batch) continue;
    const size_t o_node = pv.out.buffer.index, l_node = sum.out.buffer.index;
    if (b.is_output[o_node] || b.is_output[l_node]) continue;
    auto r_div = b.sole_reader(o_node);
    auto r_div2 = b.sole_reader(l_node);
    if (!r_div || !r_div2 || *r_div != *r_div2) continue;
    const Step& dv = b.steps[*r_div];
    if (!is_row_broadcast(dv, Op::Div) || !reads(dv.in[0], o_node) || !reads(dv.in[1], l_node)) continue;
    if (dv.rank != f1.n_batch + 2) continue;
    const Node& pv_mul = b.g.nodes[pv.nodes[0]].inner;
    const bool e_staged = pv_mul.compute_sites[0] && !pv_mul.compute_sites[0]->root;
    if (!e_staged && !fuse_always()) continue;

    Step fused;
    fused.kind = StepKind::Attention;
    fused.op = Op::Add;
    fused.rank = qk.rank;
    fused.in = {qk.in[0], qk.in[1], pv.in[1]};
    fused.out = dv.out;
    fused.form = f1;
    fused.form2 = f2;
    fused.hint = qk.hint;
    fused.hint.staged = true;
    group.insert(group.end(), ex.nodes.begin(), ex.nodes.end());
    group.insert(group.end(), pv.nodes.begin(), pv.nodes.end());
    group.insert(group.end(), sum.nodes.begin(), sum.nodes.end());
    group.insert(group.end(), dv.nodes.begin(), dv.nodes.end());
    fused.nodes = group;
    slots.push_back(i_exp);
    slots.push_back(i_pv);
    slots.push_back(i_sum);
    const size_t slot = *r_div;
    for (size_t dead : slots) b.alive[dead] = false;
    b.steps[slot] = std::move(fused);
    b.alive[slot] = true;
  }
}

// Consecutive pointwise maps over one index space become one pass: `ij-i~ij` then `^ij~ij` then
// `ij/i~ij` reads its operands once and writes once instead of moving two full-size
// intermediates through memory, which is what the reference's staged loops do for such chains
// (compiler/src/lower/node_to_stage.rs:621-674: a producer whose axes align with the consumer's
// prefix is computed inside the consumer's loops).  Fused here whatever the schedule says: the
// arithmetic per element is the same.  A link is fused when the earlier map has a single reader,
// both write the full index space in order, and every other operand is the full tensor, one value
// per row (all axes but the last), one value per column (the last axis) or a scalar.
constexpr size_t kMaxChainOps = 8, kMaxChainOperands = 4;

bool chain_operand_ok(const Access& a, size_t rank) {
  if (is_iota(a.index, rank)) return true;                        // full
  if (rank >= 1 && is_iota(a.index, rank - 1)) return true;       // per row (or scalar when rank 1)
  if (a.index.empty()) return true;                               // scalar
  return rank >= 2 && a.index.size() == 1 && a.index[0] == rank - 1;   // per column
}

void fuse_map_chains(Builder& b) {
  for (size_t n = 0; n < b.g.nodes.size(); ++n) {
    if (!b.alive[n]) continue;
    const Step& first = b.steps[n];
    if (first.kind != StepKind::Map && first.kind != StepKind::MapChain) continue;
    if (first.rank == 0 || !is_iota(first.out.index, first.rank)) continue;
    const size_t a_node = first.out.buffer.index;
    auto reader = b.sole_reader(a_node);
    if (!reader) continue;
    const Step& next = b.steps[*reader];
    if (next.kind != StepKind::Map || next.rank != first.rank || !is_iota(next.out.index, next.rank))
      continue;
    // The link: `next` reads the earlier result element for element, exactly once.
    int link = -1, links = 0;
    for (size_t i = 0; i < next.in.size(); ++i)
      if (!next.in[i].buffer.is_input && next.in[i].buffer.index == a_node) {
        link = static_cast<int>(i);
        ++links;
      }
    if (links != 1 || !is_iota(next.in[link].index, next.rank)) continue;
    bool ok = true;
    for (const Access& acc : first.in) ok = ok && chain_operand_ok(acc, first.rank);
    for (size_t i = 0; i < next.in.size(); ++i)
      if (static_cast<int>(i) != link) ok = ok && chain_operand_ok(next.in[i], next.rank);
    if (!ok) continue;

    Step fused;
    fused.kind = StepKind::MapChain;
    fused.op = next.op;
    fused.rank = first.rank;
    fused.out = next.out;
    fused.hint = next.hint;
    fused.nodes = first.nodes;
    fused.nodes.insert(fused.nodes.end(), next.nodes.begin(), next.nodes.end());
    fused.in = first.in;
    if (first.kind == StepKind::MapChain) {
      fused.chain = first.chain;
    } else {
      ChainOp op0;
      op0.op = first.op;
      op0.lhs = 0;
      op0.rhs = first.in.size() == 2 ? 1 : kChainNone;
      fused.chain = {op0};
    }
    auto operand = [&](size_t i) -> int {
      if (static_cast<int>(i) == link) return kChainPrev;
      for (size_t e = 0; e < fused.in.size(); ++e)
        if (fused.in[e].buffer == next.in[i].buffer && fused.in[e].index == next.in[i].index)
          return static_cast<int>(e);
      fused.in.push_back(next.in[i]);
      return static_cast<int>(fused.in.size() - 1);
    };
    ChainOp op1;
    op1.op = next.op;
    op1.lhs = operand(0);
    op1.rhs = next.in.size() == 2 ? operand(1) : kChainNone;
    fused.chain.push_back(op1);
    if (fused.chain.size() > kMaxChainOps || fused.in.size() > kMaxChainOperands) continue;
    const size_t slot = *reader;
    b.alive[n] = false;
    b.steps[slot] = std::move(fused);
  }
}

// A row fold whose operand is a pointwise map or chain with no other reader: the operand is
// computed inside the fold (`ij-i~ij`, `^ij~ij`, `+ij~i`), so the full-size intermediate is never
// written.  Only folds of the last axis alone, which is the split the chain's per-row and
// per-column operands are defined against.
void fuse_chain_reductions(Builder& b) {
  for (size_t n = 0; n < b.g.nodes.size(); ++n) {
    if (!b.alive[n]) continue;
    const Step& m = b.steps[n];
    if (m.kind != StepKind::Map && m.kind != StepKind::MapChain) continue;
    if (m.rank == 0 || !is_iota(m.out.index, m.rank)) continue;
    auto reader = b.sole_reader(m.out.buffer.index);
    if (!reader) continue;
    const Step& red = b.steps[*reader];
    if (red.kind != StepKind::Reduce || red.rank != m.rank || red.in.size() != 1) continue;
    if (!is_iota(red.in[0].index, red.rank) || !is_iota(red.out.index, red.rank - 1)) continue;
    bool ok = true;
    for (const Access& acc : m.in) ok = ok && chain_operand_ok(acc, m.rank);
    if (!ok || m.in.size() > kMaxChainOperands) continue;

    Step fused;
    fused.kind = StepKind::ChainReduce;
    fused.op = red.op;
    fused.rank = m.rank;
    fused.in = m.in;
    fused.out = red.out;
    fused.hint = red.hint;
    fused.nodes = m.nodes;
    fused.nodes.insert(fused.nodes.end(), red.nodes.begin(), red.nodes.end());
    if (m.kind == StepKind::MapChain) {
      fused.chain = m.chain;
    } else {
      ChainOp op0;
      op0.op = m.op;
      op0.lhs = 0;
      op0.rhs = m.in.size() == 2 ? 1 : kChainNone;
      fused.chain = {op0};
    }
    const size_t slot = *reader;
    b.alive[n] = false;
    b.steps[slot] = std::move(fused);
  }
}

// A contraction whose only reader is a pointwise map or chain over the same index space, built
// from `+ - * > <` (a bias, a scale, a rectifier) with the contraction's result as the value the
// chain starts from: the operators run in the contraction's epilogue, on the accumulator, and the
// product is never written.  The reference reaches the same with a staged producer
// (compiler/src/lower/node_to_stage.rs:621-674); here it does not depend on the schedule, because
// each element sees the same operators in the same order either way.
bool epilogue_op(Op op) {
  return op == Op::Add || op == Op::Sub || op == Op::Mul || op == Op::Max || op == Op::Min;
}

void fuse_contract_epilogues(Builder& b) {
  for (size_t n = 0; n < b.g.nodes.size(); ++n) {
    if (!b.alive[n]) continue;
    const Step& con = b.steps[n];
    if (con.kind != StepKind::Contract || !con.chain.empty()) continue;
    if (con.form.swap_out || !con.form.has_m || !con.form.has_n) continue;
    const size_t c_node = con.out.buffer.index;
    auto reader = b.sole_reader(c_node);
    if (!reader) continue;
    const Step& next = b.steps[*reader];
    if (next.kind != StepKind::Map && next.kind != StepKind::MapChain) continue;
    if (next.rank != con.out.index.size() || !is_iota(next.out.index, next.rank)) continue;
    int link = -1, links = 0;
    for (size_t i = 0; i < next.in.size(); ++i)
      if (!next.in[i].buffer.is_input && next.in[i].buffer.index == c_node) {
        link = static_cast<int>(i);
        ++links;
      }
    if (links != 1 || !is_iota(next.in[link].index, next.rank)) continue;
    std::vector<ChainOp> ops = next.chain;
    if (next.kind == StepKind::Map) {
      ChainOp op0;
      op0.op = next.op;
      op0.lhs = 0;
      op0.rhs = next.in.size() == 2 ? 1 : kChainNone;
      ops = {op0};
    }
    // The product must be the value the chain starts from and appear nowhere else; every operator
    // takes the running value on exactly one side.
    bool ok = !ops.empty() && ops.size() <= kMaxChainOps;
    std::vector<Access> others;
    std::vector<int> renumber(next.in.size(), kChainNone);
    for (size_t i = 0; ok && i < next.in.size(); ++i) {
      if (static_cast<int>(i) == link) continue;
      ok = chain_operand_ok(next.in[i], next.rank);
      renumber[i] = static_cast<int>(others.size());
      others.push_back(next.in[i]);
    }
    ok = ok && others.size() + 1 <= kMaxChainOperands;
    for (size_t j = 0; ok && j < ops.size(); ++j) {
      ChainOp& c = ops[j];
      ok = epilogue_op(c.op);
      auto is_running = [&](int code) { return j == 0 ? code == link : code == kChainPrev; };
      auto is_product = [&](int code) { return code == link; };
      const bool left = is_running(c.lhs), right = is_running(c.rhs);
      ok = ok && left != right && (c.rhs != kChainNone || left);
      if (j > 0) ok = ok && !is_product(c.lhs) && !is_product(c.rhs);
      if (!ok) break;
      auto code = [&](int x) { return is_running(x) ? kChainPrev : x == kChainNone ? x : renumber[x]; };
      c.lhs = code(c.lhs);
      c.rhs = code(c.rhs);
    }
    if (!ok) continue;

    Step fused = con;
    fused.out = Access{next.out.buffer, con.out.index};
    fused.chain = ops;
    fused.epilogue_in = others;
    fused.chain_rank = next.rank;
    fused.nodes.insert(fused.nodes.end(), next.nodes.begin(), next.nodes.end());
    const size_t slot = *reader;
    b.alive[n] = false;
    b.steps[slot] = std::move(fused);
  }
}

const char* kind_name(StepKind k) {
  switch (k) {
    case StepKind::Map: return "map";
    case StepKind::MapChain: return "map_chain";
    case StepKind::ChainReduce: return "chain_reduce";
    case StepKind::Reduce: return "reduce";
    case StepKind::Contract: return "contract";
    case StepKind::RowSoftmax: return "row_softmax";
    case StepKind::Attention: return "attention";
  }
  return "?";
}

std::string buffer_name(const Source& s) {
  return (s.is_input ? "in" : "t") + std::to_string(s.index);
}

std::string index_text(const std::vector<size_t>& idx) {
  if (idx.empty()) return ".";
  std::string out;
  for (size_t x : idx) out += std::to_string(x);
  return out;
}

}  // namespace

std::string Plan::describe() const {
  std::ostringstream os;
  os << "// i component compiled for the B200 target (sm_100a)\n";
  os << "// inputs: " << n_inputs << ", outputs: " << outputs.size() << ", kernel steps: "
     << steps.size() << "\n";
  for (size_t i = 0; i < steps.size(); ++i) {
    const Step& s = steps[i];
    os << "step " << i << ": " << kind_name(s.kind);
    if (s.kind == StepKind::Map || s.kind == StepKind::Reduce) os << " `" << op_token(s.op) << "`";
    os << "  " << buffer_name(s.out.buffer) << "[" << index_text(s.out.index) << "] <-";
    for (const auto& a : s.in) os << " " << buffer_name(a.buffer) << "[" << index_text(a.index) << "]";
    for (const auto& a : s.epilogue_in)
      os << " " << buffer_name(a.buffer) << "[" << index_text(a.index) << "]";
    os << "\n";
    switch (s.kind) {
      case StepKind::Contract:
        os << "    kernel: ib_contract (tcgen05 kind::tf32 + TMA when shapes allow, SIMT fp32 "
              "otherwise; a weighted fold in fp32 when the result has a single axis per batch entry; "
              "the k range in parts when the result has few tiles); batch axes "
           << s.form.n_batch << ", A " << (s.form.a_kmajor ? "[m,k]" : "[k,m]") << ", B "
           << (s.form.b_kmajor ? "[n,k]" : "[k,n]") << (s.form.swap_out ? ", output [n,m]" : "")
           << "\n";
        if (!s.chain.empty()) {
          os << "    epilogue (applied to each element before it is stored; a separate pass on the "
                "fp32 arm):";
          auto name = [&](int code) -> std::string {
            if (code == kChainPrev) return "_";
            return buffer_name(s.epilogue_in[code].buffer);
          };
          for (const ChainOp& c : s.chain) {
            os << "  ";
            if (c.rhs == kChainNone) os << op_token(c.op) << name(c.lhs);
            else os << name(c.lhs) << op_token(c.op) << name(c.rhs);
          }
          os << "\n";
        }
        break;
      case StepKind::RowSoftmax:
        os << "    kernel: ib_row_softmax (row resident on chip, one read + one write)\n";
        break;
      case StepKind::Attention:
        os << "    kernel: ib_attention (fused online softmax, both contractions on tcgen05, S/P/O "
              "in TMEM); batch axes "
           << s.form.n_batch << ", V " << (s.form2.b_kmajor ? "[dv,j]" : "[j,dv]");
        if (s.in.size() == 4)
          os << ", logits " << (s.op == Op::Div ? "/ " : "* ") << buffer_name(s.in[3].buffer);
        os << "\n";
        break;
      case StepKind::Reduce:
        os << "    kernel: ib_reduce\n";
        break;
      case StepKind::Map:
        os << "    kernel: ib_map\n";
        break;
      case StepKind::MapChain:
      case StepKind::ChainReduce: {
        if (s.kind == StepKind::MapChain)
          os << "    kernel: ib_map_chain (one pass):";
        else
          os << "    kernel: ib_reduce_rows_chain (fold `" << op_token(s.op) << "` of, in one pass):";
        auto name = [&](int code) -> std::string {
          if (code == kChainPrev) return "_";
          return buffer_name(s.in[code].buffer);
        };
        for (const ChainOp& c : s.chain) {
          os << "  ";
          if (c.rhs == kChainNone) os << op_token(c.op) << name(c.lhs);
          else os << name(c.lhs) << op_token(c.op) << name(c.rhs);
        }
        os << "\n";
        break;
      }
    }
    if (s.kind == StepKind::Attention || s.kind == StepKind::Contract) {
      const Geometry g = choose_geometry(s.kind, s.hint);
      os << "    geometry: 128 rows x ";
      if (s.kind == StepKind::Attention) {
        os << "128 keys per step; a row block's key range ";
        if (g.kv_granule == Geometry::kNever)
          os << "stays on one SM (row axis outermost in the schedule), no merge kernel\n";
        else
          os << "may be divided between SMs at multiples of "
             << (g.kv_granule ? (g.kv_granule + 127) / 128 * 128 : size_t(128)) << " keys"
             << (g.kv_granule ? " (the schedule's key split)\n" : "\n");
      } else {
        if (g.col_tile) os << g.col_tile << " columns (the schedule's column split)";
        else os << "128 or 256 columns by the output's width (256 rows x 256 columns per CTA pair when it has them)";
        os << " x 32 deep, 4-stage TMA ring; tiles walked ";
        if (g.col_group == Geometry::kNever) os << "row by row (row axis outermost in the schedule)\n";
        else os << "in groups of 12 column tiles\n";
      }
    }
    if (s.hint.row_split || s.hint.col_split || s.hint.staged)
      os << "    schedule: row granule " << s.hint.row_split << ", column granule "
         << s.hint.col_split << ", "
         << (s.hint.reduce_outer ? (s.kind == StepKind::Contract ? "column tiles outermost" : "reduced-axis tiles outermost")
                                 : "row tiles outermost")
         << ", " << (s.hint.staged ? "producers staged (fused)" : "producers materialised") << "\n";
    os << "    nodes:";
    for (size_t n : s.nodes) os << " n" << n;
    os << "\n";
  }
  os << "outputs:";
  for (const auto& o : outputs) os << " " << buffer_name(o);
  os << "\n";
  return os.str();
}

Geometry choose_geometry(StepKind kind, const ScheduleHint& hint) {
  Geometry g;
  const bool scheduled = hint.row_split != 0 || hint.col_split != 0;
  if (!scheduled) return g;
  if (kind == StepKind::Contract) {
    if (hint.col_split >= 256) g.col_tile = 256;
    else if (hint.col_split >= 128) g.col_tile = 128;
    if (!hint.reduce_outer) g.col_group = Geometry::kNever;   // row axis outermost: row by row
  } else if (kind == StepKind::Attention) {
    g.kv_granule = hint.reduce_outer ? hint.col_split : Geometry::kNever;
  }
  return g;
}

std::string describe_graph(const Graph& g) {
  std::ostringstream os;
  os << "graph: " << g.n_inputs << " inputs, " << g.nodes.size() << " nodes\n";
  for (size_t n = 0; n < g.nodes.size(); ++n) {
    const Node& node = g.nodes[n].inner;
    os << "  n" << n << " " << op_name(node.op) << " ";
    for (size_t i = 0; i < node.inputs.size(); ++i)
      os << (i ? "," : "") << "[" << index_text(node.inputs[i]) << "]";
    os << "~[" << index_text(node.output) << "] <-";
    for (const auto& src : g.nodes[n].inputs) os << " " << (src.is_input ? "in" : "n") << src.index;
    os << "\n";
  }
  os << "  outputs:";
  for (const auto& src : g.outputs) os << " " << (src.is_input ? "in" : "n") << src.index;
  os << "\n";
  return os.str();
}

Result<Plan> make_plan(const Graph& g) {
  Builder b(g);
  if (auto err = basic_steps(b)) return Result<Plan>::failure(*err);
  // Placements the reference's planner refuses are refused here too, before any kernel is chosen.
  if (auto err = check_schedule(g)) return Result<Plan>::failure(lower_error(*err));
  fuse_contractions(b);
  fuse_softmax(b);
  fuse_attention(b);
  fuse_deferred_attention(b);
  fuse_map_chains(b);
  fuse_chain_reductions(b);
  fuse_contract_epilogues(b);

  Plan plan;
  plan.n_inputs = g.n_inputs;
  plan.n_nodes = g.nodes.size();
  plan.outputs = g.outputs;
  for (size_t n = 0; n < g.nodes.size(); ++n)
    if (b.alive[n]) plan.steps.push_back(b.steps[n]);

  plan.input_ranks.assign(g.n_inputs, static_cast<size_t>(-1));
  for (const auto& node : g.nodes)
    for (size_t i = 0; i < node.inputs.size(); ++i)
      if (node.inputs[i].is_input) {
        size_t& r = plan.input_ranks[node.inputs[i].index];
        if (r == static_cast<size_t>(-1)) r = node.inner.inputs[i].size();
      }
  for (const auto& out : g.outputs) {
    if (out.is_input) {
      // An identity-wired output has the rank of whatever is passed in.
      plan.output_ranks.push_back(static_cast<size_t>(-1));
    } else {
      plan.output_ranks.push_back(g.nodes[out.index].inner.output.size());
    }
  }
  return Result<Plan>::success(std::move(plan));
}

}  // namespace ib
