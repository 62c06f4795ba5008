// Graph -> execution plan for the B200 target.
//
// The reference lowers a graph through a generic loop-nest planner
// (compiler/src/lower/node_to_stage.rs, stage_to_kernel_program.rs) and emits C.
// This target instead recognises the sub-graphs of the hot path and maps each
// to one hand-written kernel; anything it cannot map is a compile error (there
// is no CPU fallback).  Recognition works on canonical index numbers, never on
// axis letters, so `bhij*bhkj~bhikj` and `ik*jk~ijk` are the same contraction
// with two extra leading batch axes.
#pragma once

#include <string>
#include <vector>

#include "ir.h"

namespace ib {

enum class StepKind {
  Map,          // pointwise unary or binary, any broadcast / permutation
  MapChain,     // several pointwise operators applied in sequence in one pass
  ChainReduce,  // the same, folded along the last axis instead of stored (Step::op is the fold)
  Reduce,       // fold over the axes missing from the output
  Contract,     // Mul node + Add-reduce node = batched GEMM
  RowSoftmax,   // max, shift, exp, sum, divide over the last axis
  Attention     // Contract -> RowSoftmax -> Contract, fused online softmax
};

// One tensor access of a step: which buffer, and which step-local index each
// of its dimensions runs over.
struct Access {
  Source buffer;
  std::vector<size_t> index;
};

struct ContractForm {
  size_t n_batch = 0;          // leading axes shared by both operands and the output
  bool has_m = true, has_n = true;
  size_t m = 0, n = 0, k = 0;  // step-local index numbers
  bool a_kmajor = true;        // operand 0 stored [.., m, k]; false = [.., k, m]
  bool b_kmajor = true;        // operand 1 stored [.., n, k]; false = [.., k, n]
  bool swap_out = false;       // output stored [.., n, m]
};

// Schedule facts the kernels read (granules, loop preference, staging).
struct ScheduleHint {
  size_t row_split = 0;        // split factor on the output-row axis (0 = none)
  size_t col_split = 0;        // split factor on the reduced / column axis
  bool reduce_outer = false;   // the reduced (KV) tile loop is outermost
  bool staged = false;         // producers are staged into the consumer's loops
};

// What the schedule segment decides about a tensor-core kernel's geometry (zeros: the kernel's
// own choice, which is what a component without a schedule gets).  The reference turns splits and
// loop order into its loop nest (compiler/src/lower/node_to_stage.rs:593-692); here they select
// among the geometries the kernels have:
//   Contract   col_tile   output columns per tile: a column split of 256 or more asks for 256,
//                         one in [128, 256) for 128 (both on the single-CTA kernel); finer splits
//                         than any MMA tile leave it open (CTA pairs on 256 x 256 tiles when the
//                         output has them)
//              col_group  column tiles per raster group: with the row axis outermost in the loop
//                         order the tiles are walked row by row (every column tile in one group),
//                         with the column axis outermost in column groups of 12
//   Attention  kv_granule keys: with the key axis outermost, the key range of a block of query
//                         rows may be divided between SMs at multiples of the key split (rounded
//                         up to 128-key tiles); with the row axis outermost a row block's keys
//                         stay on one SM (kNever) and no merge kernel runs
struct Geometry {
  static constexpr size_t kNever = static_cast<size_t>(-1);
  size_t col_tile = 0, col_group = 0, kv_granule = 0;
};
Geometry choose_geometry(StepKind kind, const ScheduleHint& hint);


// One operator of a MapChain.  Operand codes: kChainNone (unary form), kChainPrev (the result of
// the operator before it), or an index into Step::in.
constexpr int kChainNone = -1;
constexpr int kChainPrev = -2;
struct ChainOp {
  Op op = Op::Add;
  int lhs = kChainNone, rhs = kChainNone;
};

struct Step {
  StepKind kind = StepKind::Map;
  Op op = Op::Add;
  size_t rank = 0;                 // size of the step-local index space
  std::vector<Access> in;
  Access out;                      // out.buffer.index = node that owns the result
  ContractForm form;               // Contract; Attention uses form (QK) and form2 (PV)
  ContractForm form2;
  ScheduleHint hint;
  std::vector<size_t> nodes;       // graph nodes folded into this step
  std::vector<ChainOp> chain;      // MapChain: the operators in order
  // Contract with pointwise operators applied to its result before it is stored: `chain` holds
  // them (kChainPrev in the first is the contraction's result, other codes index `epilogue_in`),
  // `epilogue_in` their other operands, indexed over the result's own axes 0 .. chain_rank - 1.
  std::vector<Access> epilogue_in;
  size_t chain_rank = 0;
};

struct Plan {
  size_t n_inputs = 0;
  size_t n_nodes = 0;
  std::vector<Step> steps;
  std::vector<Source> outputs;
  std::vector<size_t> output_ranks;
  // For every graph input: its rank as implied by the patterns that read it.
  std::vector<size_t> input_ranks;
  std::string describe() const;    // text returned by i_code
};

Result<Plan> make_plan(const Graph& g);

// schedule.cc — the reference's message when its loop-nest planner would refuse the graph's
// compute-at placements (mismatched splits between a staged producer and its consumer, an online
// reduction whose correction no accumulator absorbs); nothing when it would accept them.
std::optional<std::string> check_schedule(const Graph& g);

// Text form of the wired graph: one line per node (op, index patterns, sources)
// and the output list.  Printed by i_code ahead of the plan.
std::string describe_graph(const Graph& g);

}  // namespace ib
