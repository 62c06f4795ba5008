// Fused online-softmax attention O = softmax(Q K^T) V on sm_100a tensor cores.
//
// This is the B200 form of the one kernel the reference emits for
// `mm_t >> row_max_shift >> exp >> row_normalize >> mm`
// (ilang-python/annotated-flashattn.c:52-310): per KV tile it forms S = Q K^T,
// updates the running row maximum m and row sum l, and accumulates
// O += exp(S - m) V with O rescaled when m moves.  The reference divides P by
// the running sum in every tile and multiplies O by l_old/l_new (:186-275);
// dividing once at the end is the same quantity.  exp is powf(2.71828175f, x)
// in the reference; here it is 2^(x * log2(2.71828175)).
//
// Four instantiations (enum Arm): both contractions on TF32 operands; both on
// bf16 operands; S = Q K^T on TF32 operands and O += P V on fp16 operands (same
// 10-bit mantissa, V scaled per head by a power of two into fp16's range, P in
// [0, 1]); or, the default for large problems, both on fp16 operands, with Q
// scaled per row and K per tile of 128 keys as well and the scales multiplied
// back into the factor that takes S to the exponent.  With 16-bit P the softmax
// warps pack two probabilities per tensor-memory column.
//
// Two kernels.  The arms with 32-bit operands (TF32, and TF32 x fp16) run the one described
// here; the 16-bit arms run attention_pipelined_kernel further down, described there.
// One CTA (384 threads) owns 128 query rows and walks the keys in tiles of 128:
//   warp 0      TMA producer: K tiles ([128 keys][d]) and V^T tiles
//               ([dv][128 keys]) as 128-byte-swizzled rows through a ring of
//               three 64 KB slots.
//   warp 1      MMA issuer.  Both contractions take their A operand from
//               tensor memory (measured on B200: an M=128 tcgen05.mma with A
//               in shared memory never costs less than ~124 cycles, with A in
//               tensor memory ~71 for N=128, against 64 ideal):
//               S = Q K^T with Q resident in tensor memory for the whole
//               kernel, O += P V with P read where the softmax wrote it.  S is
//               double-buffered so Q K^T of the next tile overlaps the softmax
//               of this one.
//   warps 4-11  softmax: two warpgroups share every row, warpgroup h taking
//               key columns [64h, 64h+64) of the tile (a warp can only reach
//               its own 32-lane quadrant of tensor memory, so rows cannot be
//               split).  The halves of the row maximum meet through shared
//               memory and a 256-thread named barrier; each half keeps its own
//               partial row sum until the end.  O is rescaled in tensor memory
//               only when the maximum grows by more than 2^8.
// Tensor memory (512 columns): Q 128 | S buffer 0 128 | S buffer 1 128 | O 128.
// Q is loaded from global memory by the softmax threads, rounded to the operand
// type and stored to tensor memory once per row tile: for the first row tile of a
// CTA at kernel start, for every later one as soon as the last Q K^T of the row
// tile before has been consumed, i.e. before that row tile's O is read out, so
// the next Q K^T overlaps the read-out.  K/V rows past the end are zero-filled by
// TMA and masked to -inf; query rows past the end are computed and not stored.
//
// Work is balanced over the SMs.  CTA g of G first takes whole row tiles
// g, g+G, g+2G, ... (neighbouring CTAs then stream the same head's K/V at the
// same time, which keeps them in L2).  The row tiles left over when their number
// is not a multiple of G are split stream-K style: their (row tile, key tile)
// pairs form one flat sequence cut into G equal contiguous ranges.  A range
// piece that does not cover its row tile completely is written as a normalised
// partial O with its (m, l); a small second kernel merges the pieces.
// Roofline: tensor-bound, 4*Nq*Nk*d FLOP per head.
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace ib {
namespace {

using namespace sm100;

constexpr int kBQ = 128;           // query rows per CTA
constexpr int kBKV = 128;          // keys per KV tile
constexpr int kThreads = 384;
constexpr int kThreadsPipelined = 512;    // roles, statistics, and two softmax warpgroups
constexpr int kChunkBytes = 128 * 128;     // 128 rows of 128 bytes: 32 fp32 or 64 bf16 per row
constexpr int kMaxRing = 6;

// Arithmetic of the two contractions.  MIXED runs S = Q K^T on TF32 operands and O += P V on
// fp16 ones: fp16 has TF32's 10-bit mantissa, P lies in [0, 1], and V is scaled per head by a
// power of two into fp16's range, so the result has TF32 accuracy while the second contraction
// issues half as many MMAs.  F16 does the same for S = Q K^T: Q is scaled per query row and K per
// tile of 128 keys by powers of two into fp16's range (the scales return, exactly, in the
// multiplier that takes S to the exponent), so both contractions issue half as many MMAs on
// operands of TF32's precision.
enum class Arm { TF32, BF16, MIXED, F16 };

// Per contraction: a tile of 128 keys is 4 chunks of 32 fp32 or 2 chunks of 64 16-bit
// elements; the ring always has three slots (the producer's slot-reuse waits rely on that
// distance, see there).  One MMA consumes 32 bytes of every operand row (8 fp32 or 16 16-bit
// values along K) and 8 tensor-memory columns of its A operand (16-bit pairs are packed two to
// a column), so a 128-deep contraction is 16 or 8 instructions.
template <Arm ARM>
struct Geometry {
  static constexpr bool kQkHalf = ARM == Arm::BF16 || ARM == Arm::F16;   // Q, K are 16-bit
  static constexpr bool kPvHalf = ARM != Arm::TF32;               // P, V are 16-bit
  static constexpr bool kScaledQk = ARM == Arm::F16;              // Q rows and K tiles carry scales
  static constexpr Fmt kQkFmt = ARM == Arm::BF16 ? Fmt::BF16 : (ARM == Arm::F16 ? Fmt::F16 : Fmt::TF32);
  static constexpr Fmt kPvFmt = ARM == Arm::TF32 ? Fmt::TF32 : (ARM == Arm::BF16 ? Fmt::BF16 : Fmt::F16);
  static constexpr int kQkChunkElems = kQkHalf ? 64 : 32;
  static constexpr int kQkStepElems = kQkHalf ? 16 : 8;           // K per MMA
  static constexpr int kQkSteps = 128 / kQkStepElems;             // 16 or 8
  static constexpr int kPvChunkElems = kPvHalf ? 64 : 32;
  static constexpr int kPvTileChunks = 128 / kPvChunkElems;       // 4 or 2
  static constexpr int kPvSteps = kPvHalf ? 8 : 16;
  static constexpr int kSlotBytes = (kQkHalf && kPvHalf ? 2 : 4) * kChunkBytes;   // 32 KB or 64 KB
  static constexpr int kRing = 3;
};
constexpr int kRingBytes = 3 * 4 * kChunkBytes;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemQ = 0;
constexpr uint32_t kTmemS = 128;           // + buf * 128
constexpr uint32_t kTmemO = 384;
constexpr float kLog2E32 = 1.4426950216293335f;  // log2(2.71828175f)
constexpr float kRescaleThreshold = 8.0f;

struct Params {
  const float* q;      // [batch][nq][d], original fp32
  int nq, nk, d, dv, batch;
  int q_tiles;         // 128-row tiles per head
  int kv_tiles;        // 128-key tiles per head
  int ctas;               // G
  int full_waves;         // whole row tiles every CTA takes before the tail
  int coarse;          // key tiles per granule: a row tile's keys are divided among CTAs only at
  int kv_coarse;       // multiples of it; kv_coarse = granules per row tile (the last may be short)
  long long iters_base;   // tail (row tile, granule) pairs per CTA: CTA g takes iters_base, plus
  int iters_rem;          // one more when g < iters_rem
  const float* v_scale;   // mixed arm: V^T holds V / v_scale[head] (a power of two); else null
  const float* k_tile_scale;  // fp16 arm: K holds K / k_tile_scale[head][key tile] (powers of two)
  const float* logit_scale;   // one value on the device, or null: the logits are S * it (S / it when
  int logit_divide;           // logit_divide), applied to Q as it is staged
  float* o;            // [batch][nq][dv]
  float* part_o;       // [2 * ctas][128][dv]: slot 2g + (0: first piece, 1: last piece of CTA g)
  float* part_m;       // [2 * ctas][128]
  float* part_l;
  int* status;
  unsigned long long* prof;   // optional per-CTA wait-cycle counters (debugging aid), or null
};

struct Shared {
  uint64_t kv_full[kMaxRing];
  uint64_t q_ready;
  uint64_t o_free;           // the epilogue of a piece has read O
  uint64_t s_full[4];        // [tile & 1] in the first kernel, [tile & 3] in the pipelined one
  uint64_t p_full[2];
  uint64_t pv_done[4];       // likewise; see the note at its wait
  uint64_t s_free[2];        // pipelined kernel: the softmax warps have read S[buf] into registers
  uint32_t tmem_slot;
  AbortState abort;
  int give_up;               // raised before a named barrier, read after it
  float pub_m[4][kBQ];       // reference maximum per row for a tile, from the statistics warps
  float row_mul[2][kBQ];     // [piece & 1]: log2(e) x the row's Q scale, for the statistics warps
  float half_max[2][2][kBQ]; // [iteration parity][warpgroup][row]
  float half_sum[2][kBQ];
  float q_absmax[2][kBQ];    // pipelined kernel: the two column halves' shares of a Q row's largest magnitude
  uint64_t m_ready[4];       // pipelined kernel: [tile & 3], the tile's reference maximum is published
};

// One contiguous run of key tiles of one row tile.
struct Piece {
  int unit;        // row tile index over the whole call (head * q_tiles + tile)
  int kv_lo, n_kv;
  bool whole;      // covers every key tile: the result is final
  int ordinal;     // 0 = first tail piece of this CTA, 1 = a later one
};

// Walks this CTA's pieces.  The tail position is kept as (row tile, key tile) and advanced by
// additions: the one division happens in pieces_begin, not per piece (every role of the CTA walks
// the sequence, some of them twice to look one piece ahead).
struct PieceCursor {
  int wave;
  int tail_unit;     // row tile (within the tail) of the next piece
  int kv_lo;         // its first granule of key tiles
  int remaining;     // (row tile, granule) pairs of the tail still to hand out
  bool first;
};

__device__ __forceinline__ PieceCursor pieces_begin(const Params& p) {
  PieceCursor c;
  const int g = static_cast<int>(blockIdx.x);
  c.wave = 0;
  const long long lo = g * p.iters_base + min(g, p.iters_rem);
  c.tail_unit = static_cast<int>(lo / p.kv_coarse);
  c.kv_lo = static_cast<int>(lo - static_cast<long long>(c.tail_unit) * p.kv_coarse);
  c.remaining = static_cast<int>(p.iters_base) + (g < p.iters_rem ? 1 : 0);
  c.first = true;
  return c;
}

// Every role of a CTA walks the same sequence of pieces.
__device__ __forceinline__ bool next_piece(const Params& p, PieceCursor& c, Piece& out) {
  if (c.wave < p.full_waves) {
    out.unit = c.wave * p.ctas + static_cast<int>(blockIdx.x);
    out.kv_lo = 0;
    out.n_kv = p.kv_tiles;
    out.whole = true;
    out.ordinal = 0;
    ++c.wave;
    return true;
  }
  if (c.remaining <= 0) return false;
  out.unit = p.full_waves * p.ctas + c.tail_unit;
  const int granules = min(p.kv_coarse - c.kv_lo, c.remaining);
  out.kv_lo = c.kv_lo * p.coarse;
  out.n_kv = min(p.kv_tiles - out.kv_lo, granules * p.coarse);
  out.whole = c.kv_lo == 0 && granules == p.kv_coarse;
  out.ordinal = c.first ? 0 : 1;
  c.first = false;
  c.remaining -= granules;
  c.kv_lo += granules;
  if (c.kv_lo == p.kv_coarse) {
    c.kv_lo = 0;
    ++c.tail_unit;
  }
  return true;
}


// Two floats -> one 32-bit word of bf16 (round to nearest even), first value in the low half.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t out;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
  return out;
}

// The power of two that brings a largest magnitude into [2^14, 2^15) (1 for zero, inf or NaN):
// what fp16 operands are stored over so that large values fit and small ones keep their mantissa.
__device__ __forceinline__ float f16_range_scale(float absmax) {
  if (!(absmax > 0.0f) || !(absmax < CUDART_INF_F)) return 1.0f;
  int e;
  frexpf(absmax, &e);                          // absmax = f * 2^e, f in [0.5, 1)
  return ldexpf(1.0f, max(e - 15, -120));
}

__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t out;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
  return out;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

// Two fp16 exponentials (2^x) in one special-function instruction.
__device__ __forceinline__ uint32_t ex2_f16x2(uint32_t x) {
  uint32_t y;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t add_f16x2(uint32_t a, uint32_t b) {
  uint32_t y;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(y) : "r"(a), "r"(b));
  return y;
}
__device__ __forceinline__ float f16_lo(uint32_t pair) {
  float y;
  asm("{.reg .f16 lo, hi; mov.b32 {lo, hi}, %1; cvt.f32.f16 %0, lo;}" : "=f"(y) : "r"(pair));
  return y;
}
__device__ __forceinline__ float f16_hi(uint32_t pair) {
  float y;
  asm("{.reg .f16 lo, hi; mov.b32 {lo, hi}, %1; cvt.f32.f16 %0, hi;}" : "=f"(y) : "r"(pair));
  return y;
}
#ifndef IB_ATTN_HALF_EXP
#define IB_ATTN_HALF_EXP 1
#endif
constexpr bool kHalfExp = IB_ATTN_HALF_EXP != 0;

// Per-phase cycle counters (written to Params::prof) exist only in builds with
// -DIB_ATTN_PROFILE=1; the shipped library compiles them out.
#ifndef IB_ATTN_PROFILE
#define IB_ATTN_PROFILE 0
#endif
constexpr bool kProf = IB_ATTN_PROFILE != 0;

template <bool PROF>
__device__ __forceinline__ long long tick() {
  return PROF ? clock64() : 0ll;
}

__device__ __forceinline__ void softmax_pair_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}


// Q of one row tile: global -> operand type (nearest) -> tensor memory, this thread's 64
// features [64h, 64h+64) of its row; then one arrival per warp on q_ready.
// Returns the factor that takes this row's S to the exponent's units, K's tile scale aside:
// log2(e), times the row's own power of two where Q is stored scaled.
template <Arm ARM>
__device__ __forceinline__ float stage_q_rows(const Params& p, Shared* sh, uint32_t tmem_q, int head,
                                              int q_tile, int r, int h, int lane, int piece = -1) {
  using G = Geometry<ARM>;
  float row_mul = kLog2E32;
  const long long row = static_cast<long long>(q_tile) * kBQ + r;
  const float* qrow = p.q + (static_cast<size_t>(head) * p.nq + row) * p.d;
  const bool live = row < p.nq;
  const bool vec = (reinterpret_cast<uintptr_t>(p.q) & 15u) == 0 && p.d % 4 == 0;
  // A scale on the logits is a scale on Q: (c q) . k = c (q . k).  Read here, once per row
  // tile, rather than held in a register across the key loop.
  float qs = 1.0f;
  if (p.logit_scale) {
    qs = __ldg(p.logit_scale);
    if (p.logit_divide) qs = 1.0f / qs;
  }
  // This thread's 64 features [64h, 64h+64) of its row, rounded to the operand type.
  auto load4 = [&](int col) {
    float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (live && vec && col + 4 <= p.d) {
      x = *reinterpret_cast<const float4*>(qrow + col);
    } else if (live) {
      if (col + 0 < p.d) x.x = qrow[col + 0];
      if (col + 1 < p.d) x.y = qrow[col + 1];
      if (col + 2 < p.d) x.z = qrow[col + 2];
      if (col + 3 < p.d) x.w = qrow[col + 3];
    }
    x.x *= qs; x.y *= qs; x.z *= qs; x.w *= qs;
    return x;
  };
  static_assert(!G::kQkHalf, "the 16-bit arms stage Q with stage_q_half");
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int col0 = h * 64 + c * 32;
    uint32_t v[32];
#pragma unroll
    for (int e = 0; e < 32; e += 4) {
      const float4 x = load4(col0 + e);
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v[e + 0]) : "f"(x.x));
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v[e + 1]) : "f"(x.y));
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v[e + 2]) : "f"(x.z));
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v[e + 3]) : "f"(x.w));
    }
    tmem_st_32x32(tmem_q + col0, v);
  }
  (void)piece;
  tmem_wait_st();
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(&sh->q_ready);
  return row_mul;
}

// End of a piece on the softmax warps: waits for the last P V, adds the two halves of the row
// sum, normalises and stores this thread's columns [64h, 64h+64) of O (to the output, or to the
// partial slot with its (m, l) when the piece covers only part of the keys).
__device__ __forceinline__ void finish_piece(const Params& p, Shared* sh, uint32_t o_tmem, int h,
                                             int r, long long row, int b, bool whole, int part_slot,
                                             float l, float m_used, int dv_chunks,
                                             uint64_t* last_pv_done, uint32_t last_parity,
                                             bool& dead) {
  if (!sh->give_up && !dead)
    dead = !mbar_wait_warp(last_pv_done, last_parity, &sh->abort, p.status, 209);
  sh->half_sum[h][r] = l;
  if (dead) sh->give_up = 1;
  softmax_pair_sync();
  if (sh->give_up) return;
  tc_fence_after_sync();
  const float l_total = l + sh->half_sum[h ^ 1][r];
  const float inv = (p.v_scale ? p.v_scale[b] : 1.0f) / l_total;
  float* dst;
  if (whole) {
    dst = p.o + (static_cast<size_t>(b) * p.nq + row) * p.dv;
  } else {
    const size_t prow = static_cast<size_t>(part_slot) * kBQ + r;
    dst = p.part_o + prow * p.dv;
    if (h == 0) {
      p.part_m[prow] = m_used;
      p.part_l[prow] = l_total;
    }
  }
  const bool vec_ok = (p.dv % 4 == 0) && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
  for (int c = h * 2; c < h * 2 + 2 && c < dv_chunks; ++c) {
    uint32_t o[32];
    tmem_ld_32x32(o_tmem + c * 32, o);
    tmem_wait_ld();
    if (row < p.nq || !whole) {
      if (vec_ok && c * 32 + 32 <= p.dv) {
#pragma unroll
        for (int v = 0; v < 8; ++v)
          *reinterpret_cast<float4*>(dst + c * 32 + 4 * v) = make_float4(
              __uint_as_float(o[4 * v]) * inv, __uint_as_float(o[4 * v + 1]) * inv,
              __uint_as_float(o[4 * v + 2]) * inv, __uint_as_float(o[4 * v + 3]) * inv);
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (c * 32 + e < p.dv) dst[c * 32 + e] = __uint_as_float(o[e]) * inv;
      }
    }
  }
}

// TMA producer (one thread): streams the K and V^T tiles of this CTA's pieces through the
// three-slot ring, in the order the MMA thread consumes them.
template <Arm ARM>
__device__ __forceinline__ void run_producer(const CUtensorMap* map_k, const CUtensorMap* map_vt,
                                             const Params& p, Shared* sh, uint8_t* ring) {
  using G = Geometry<ARM>;
  constexpr int kRing = G::kRing;
  constexpr int kSlotBytes = G::kSlotBytes;
  constexpr int kBarMask = 1;
  constexpr int kBarShift = 1;
  AbortState* abort = &sh->abort;
  const int d_chunks = (p.d + G::kQkChunkElems - 1) / G::kQkChunkElems;
  tma_prefetch_descriptor(map_k);
  tma_prefetch_descriptor(map_vt);
  // K and V^T come from the preparation kernel before this one in the stream;
  // this thread is the only one that reads them (Q, read by the softmax warps,
  // is an input of the call and older than that kernel).
  grid_dependency_wait();
  int slot = 0;
  bool ok = true;
  long long waited = 0;
  int b = 0;
  // A ring slot is free again when the MMAs that read its tile have completed:
  // Q K^T of tile t for a K tile (signalled on s_full[t & 1]), P V of tile t for
  // a V tile (pv_done[t & 1]); t counts this CTA's key tiles.  The producer
  // remembers who occupies each slot and waits for that event before reuse.  It
  // meets every event once and in order.  A parity wait must never be two phases
  // behind: with three slots and two barriers the next-but-one event on the same
  // barrier needs a tile this producer has not loaded yet (K(t) and K(t + 2) are
  // four loads apart).
  uint64_t* occupant_bar[kRing] = {};
  uint32_t occupant_parity[kRing] = {};
  long long tile_k = 0, tile_v = 0;       // tile counters of the next K / V load
  auto acquire = [&](int code) {
    if (!occupant_bar[slot]) return;
    const long long t0 = tick<kProf>();
    ok = mbar_wait(occupant_bar[slot], occupant_parity[slot], abort, p.status, code);
    waited += tick<kProf>() - t0;
  };
  auto load_k = [&](int j) {
    acquire(201);
    if (!ok) return;
    uint8_t* dst = ring + slot * kSlotBytes;
    mbar_arrive_expect_tx(&sh->kv_full[slot], d_chunks * kChunkBytes);
    for (int c = 0; c < d_chunks; ++c)
      tma_load_3d(dst + c * kChunkBytes, map_k, &sh->kv_full[slot], c * G::kQkChunkElems,
                  j * kBKV, b);
    occupant_bar[slot] = &sh->s_full[tile_k & kBarMask];
    occupant_parity[slot] = static_cast<uint32_t>((tile_k >> kBarShift) & 1);
    ++tile_k;
    if (++slot == kRing) slot = 0;
  };
  auto load_v = [&](int j) {
    acquire(202);
    if (!ok) return;
    uint8_t* dst = ring + slot * kSlotBytes;
    mbar_arrive_expect_tx(&sh->kv_full[slot], G::kPvTileChunks * kChunkBytes);
    for (int c = 0; c < G::kPvTileChunks; ++c)
      tma_load_3d(dst + c * kChunkBytes, map_vt, &sh->kv_full[slot],
                  j * kBKV + c * G::kPvChunkElems, 0, b);
    occupant_bar[slot] = &sh->pv_done[tile_v & kBarMask];
    occupant_parity[slot] = static_cast<uint32_t>((tile_v >> kBarShift) & 1);
    ++tile_v;
    if (++slot == kRing) slot = 0;
  };
  // Per piece, consumption order is K(0), then per tile K(j+1) before V(j).
  PieceCursor cursor = pieces_begin(p);
  Piece pc;
  const bool q_prefetchable = (reinterpret_cast<uintptr_t>(p.q) & 15u) == 0;
  while (ok && next_piece(p, cursor, pc)) {
    b = pc.unit / p.q_tiles;
    {
      // Pull the Q rows of the piece after this one into L2 while this one runs.
      PieceCursor ahead = cursor;
      Piece nx;
      if (q_prefetchable && next_piece(p, ahead, nx) && nx.unit != pc.unit) {
        const int nb = nx.unit / p.q_tiles;
        const long long row0 = static_cast<long long>(nx.unit - nb * p.q_tiles) * kBQ;
        const long long rows = min(static_cast<long long>(kBQ), p.nq - row0);
        prefetch_l2_bulk(p.q + (static_cast<size_t>(nb) * p.nq + row0) * p.d,
                         static_cast<uint32_t>(rows * p.d * 4));
      }
    }
    constexpr int kAhead = 1;
    for (int jj = 0; ok && jj < kAhead && jj < pc.n_kv; ++jj) load_k(pc.kv_lo + jj);
    for (int jj = 0; ok && jj < pc.n_kv; ++jj) {
      if (jj + kAhead < pc.n_kv) load_k(pc.kv_lo + jj + kAhead);
      if (ok) load_v(pc.kv_lo + jj);
    }
  }
  if (kProf && p.prof) p.prof[blockIdx.x * 16 + 0] = waited;
}

template <Arm ARM>
__global__ void __launch_bounds__(kThreads, 1)
attention_tf32_kernel(const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_vt, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  using G = Geometry<ARM>;
  constexpr int kRing = G::kRing;
  constexpr int kSlotBytes = G::kSlotBytes;
  uint8_t* ring = smem;                                     // [kRing][kSlotBytes]
  Shared* sh = reinterpret_cast<Shared*>(ring + kRingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int d_chunks = (p.d + G::kQkChunkElems - 1) / G::kQkChunkElems;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&sh->kv_full[s], 1);
    }
    mbar_init(&sh->q_ready, 8);            // one arrival per softmax warp
    mbar_init(&sh->o_free, 8);
    for (int u = 0; u < 2; ++u) {
      mbar_init(&sh->s_full[u], 1);
      mbar_init(&sh->p_full[u], 8);
      mbar_init(&sh->pv_done[u], 1);
    }
    sh->abort.flag = 0;
    sh->give_up = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_slot, kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_slot;
  AbortState* abort = &sh->abort;
  // The merge kernel that follows may be scheduled from now on (it waits for this
  // grid to finish before it reads anything).
  trigger_dependent_launch();

  if (warp == 0) {
    if (lane == 0) run_producer<ARM>(&map_k, &map_vt, p, sh, ring);
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_fmt(G::kQkFmt, kBQ, kBKV);
      const uint32_t n_pv = static_cast<uint32_t>((p.dv + 15) / 16 * 16);
      const uint32_t idesc_pv = make_idesc_fmt(G::kPvFmt, kBQ, n_pv);
      const int k_steps = (p.d + G::kQkStepElems - 1) / G::kQkStepElems;
      int slot = 0;
      uint32_t phase = 0;
      const uint32_t ring_addr = smem_u32(ring);
      long long wait_k = 0, wait_v = 0, wait_p = 0, wait_q = 0, issue_qk_cycles = 0, issue_pv_cycles = 0;
      const long long t_start = tick<kProf>();
      bool ok = true;
      long long it = 0;                       // key tiles issued so far by this CTA

      // S[buf] = Q K^T from the K tile in the current slot (A = Q in tensor memory).
      auto issue_qk = [&](int buf) {
        const long long t0 = tick<kProf>();
        if (!(ok = mbar_wait(&sh->kv_full[slot], phase, abort, p.status, 204))) return;
        wait_k += tick<kProf>() - t0;
        tc_fence_after_sync();
        // One descriptor per slot; a K step moves it by a compile-time constant
        // (32 bytes inside the swizzled row, 16 KB to the next 32-feature chunk),
        // so the issuing thread spends one 64-bit add per MMA.
        const long long ti = tick<kProf>();
        const uint64_t k_desc = make_smem_desc_sw128(ring_addr + slot * kSlotBytes);
        const uint32_t d_tmem = tmem_base + kTmemS + static_cast<uint32_t>(buf * kBKV);
        const uint32_t q_tmem = tmem_base + kTmemQ;
#pragma unroll
        for (int ks = 0; ks < G::kQkSteps; ++ks) {
          if (ks < k_steps)
            mma_ts_w<G::kQkHalf>(d_tmem, q_tmem + ks * 8,
                         k_desc + (((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4), idesc_qk,
                         ks != 0 ? 1u : 0u);
        }
        mma_commit(&sh->s_full[buf]);          // S ready, and the K tile's slot is free
        issue_qk_cycles += tick<kProf>() - ti;
        if (++slot == kRing) { slot = 0; phase ^= 1; }
      };
      // O += P[buf] V from the V^T tile in the current slot (A = P in tensor memory).
      auto issue_pv = [&](long long t, bool first_of_piece, int piece) {
        const int buf = static_cast<int>(t & 1);
        long long t0 = tick<kProf>();
        if (!(ok = mbar_wait(&sh->kv_full[slot], phase, abort, p.status, 205))) return;
        // The first P V of a piece overwrites O: the piece before must have read it out.
        if (first_of_piece && piece > 0 &&
            !(ok = mbar_wait(&sh->o_free, static_cast<uint32_t>((piece - 1) & 1), abort, p.status, 210)))
          return;
        wait_v += tick<kProf>() - t0;
        t0 = tick<kProf>();
        if (!(ok = mbar_wait(&sh->p_full[buf], (t >> 1) & 1, abort, p.status, 206))) return;
        wait_p += tick<kProf>() - t0;
        tc_fence_after_sync();
        const long long ti = tick<kProf>();
        const uint64_t v_desc = make_smem_desc_sw128(ring_addr + slot * kSlotBytes);
        const uint32_t d_tmem = tmem_base + kTmemO;
        const uint32_t p_tmem = tmem_base + kTmemS + static_cast<uint32_t>(buf * kBKV);
        // Keys 64h..64h+63 of P sit at the start of softmax half h's 64 columns:
        // 64 columns of fp32 (TF32) or 32 columns of packed bf16 pairs.
        auto p_col = [&](int ks) -> uint32_t {
          constexpr int kHalfSteps = G::kPvSteps / 2;
          return p_tmem + static_cast<uint32_t>((ks / kHalfSteps) * 64 + (ks % kHalfSteps) * 8);
        };
        if (first_of_piece) {
          mma_ts_w<G::kPvHalf>(d_tmem, p_col(0), v_desc, idesc_pv, 0u);
        } else {
          mma_ts_w<G::kPvHalf>(d_tmem, p_col(0), v_desc, idesc_pv, 1u);
        }
#pragma unroll
        for (int ks = 1; ks < G::kPvSteps; ++ks)
          mma_ts_w<G::kPvHalf>(d_tmem, p_col(ks),
                       v_desc + (((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4), idesc_pv, 1u);
        mma_commit(&sh->pv_done[buf]);         // O updated, and the V tile's slot is free
        issue_pv_cycles += tick<kProf>() - ti;
        if (++slot == kRing) { slot = 0; phase ^= 1; }
      };

      PieceCursor cursor = pieces_begin(p);
      Piece pc;
      for (int piece = 0; ok && next_piece(p, cursor, pc); ++piece) {
        const int n_kv = pc.n_kv;
        // Q of this piece is in tensor memory.
        const long long tq = tick<kProf>();
        if (!(ok = mbar_wait(&sh->q_ready, piece & 1, abort, p.status, 203))) break;
        wait_q += tick<kProf>() - tq;
        tc_fence_after_sync();
        issue_qk(static_cast<int>(it & 1));
        for (int jj = 0; ok && jj < n_kv; ++jj) {
          if (jj + 1 < n_kv) issue_qk(static_cast<int>((it + jj + 1) & 1));
          if (ok) issue_pv(it + jj, jj == 0, piece);
        }
        it += n_kv;
      }
      if (kProf && p.prof) {
        p.prof[blockIdx.x * 16 + 1] = wait_k;
        p.prof[blockIdx.x * 16 + 2] = wait_v;
        p.prof[blockIdx.x * 16 + 5] = issue_qk_cycles;
        p.prof[blockIdx.x * 16 + 6] = issue_pv_cycles;
        p.prof[blockIdx.x * 16 + 3] = wait_p;
        p.prof[blockIdx.x * 16 + 4] = tick<kProf>() - t_start;
        p.prof[blockIdx.x * 16 + 8] = wait_q;
      }
    }
  } else if (warp >= 4) {
    const int h = (warp - 4) >> 2;            // column half of this warpgroup
    const int quad = warp & 3;                // TMEM lane quadrant
    const int r = quad * 32 + lane;           // row within the tile
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t o_tmem = tmem_base + lane_bits + kTmemO;
    const int dv_chunks = (p.dv + 31) / 32;
    long long it = 0;                         // key tiles consumed so far by this CTA
    long long wait_s = 0;
    long long c_load = 0, c_max = 0, c_sync = 0, c_exp = 0, c_store = 0;   // PROF: cycles per phase
    const long long t_start = tick<kProf>();
    bool dead = false;                        // a wait gave up; keep hitting the barriers only
    float row_mul = kLog2E32;                 // S of this thread's row -> exponent units (see stage_q)

    const uint32_t tmem_q = tmem_base + lane_bits + kTmemQ;   // this quadrant's rows of Q
    auto stage_q = [&](int head, int q_tile) -> float {
      return stage_q_rows<ARM>(p, sh, tmem_q, head, q_tile, r, h, lane);
    };

    PieceCursor cursor = pieces_begin(p);
    Piece pc;
    bool first_piece = true;
    while (next_piece(p, cursor, pc)) {
    const int kv_lo = pc.kv_lo, n_kv = pc.n_kv;
    const int b = pc.unit / p.q_tiles;
    const int qt = pc.unit - b * p.q_tiles;
    const long long row = static_cast<long long>(qt) * kBQ + r;
    const bool whole = pc.whole;
    const int part_slot = 2 * static_cast<int>(blockIdx.x) + pc.ordinal;

    if (first_piece) row_mul = stage_q(b, qt);   // later pieces: staged at the end of the piece before
    first_piece = false;

    float ks_ahead = 1.0f;                    // fp16 arm: the next tile's K scale, read a tile early
    float m_used = -CUDART_INF_F;             // running maximum, log2 domain
    float l = 0.0f;                           // this half's share of the row sum

    for (int jj = 0; jj < n_kv; ++jj) {
      const long long t = it + jj;            // position in this CTA's sequence of key tiles
      const int buf = static_cast<int>(t & 1);
      const uint32_t s_tmem = tmem_base + lane_bits + kTmemS + static_cast<uint32_t>(buf * kBKV) +
                              static_cast<uint32_t>(h * 64);
      uint32_t s0[32], s1[32];
      if (!dead) {
        const long long t0 = tick<kProf>();
        dead = !mbar_wait_warp(&sh->s_full[buf], (t >> 1) & 1, abort, p.status, 207);
        wait_s += tick<kProf>() - t0;
      }
      // S -> exponent units: log2(e), times the scales Q's row and K's tile were stored over.
      // K's scales come from the preparation kernel; every read of them follows an S that was
      // computed from its K, so the kernel has completed.
      float mul = kLog2E32;
      if (G::kScaledQk) {
        const float* ks = p.k_tile_scale + static_cast<size_t>(b) * p.kv_tiles + kv_lo + jj;
        const float here = jj == 0 ? __ldg(ks) : ks_ahead;
        if (jj + 1 < n_kv) ks_ahead = __ldg(ks + 1);
        mul = row_mul * here;
      }
      float mx = -CUDART_INF_F;
      long long tp = tick<kProf>();
      if (!dead) {
        tc_fence_after_sync();
        tmem_ld_32x32(s_tmem, s0);
        tmem_ld_32x32(s_tmem + 32, s1);
        tmem_wait_ld();
        c_load += tick<kProf>() - tp;
        tp = tick<kProf>();
        const int col0 = (kv_lo + jj) * kBKV + h * 64;
        if (col0 + 64 > p.nk) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (col0 + c >= p.nk) s0[c] = __float_as_uint(-CUDART_INF_F);
            if (col0 + 32 + c >= p.nk) s1[c] = __float_as_uint(-CUDART_INF_F);
          }
        }
        // Three-operand maximum: 32 instructions for the 64 values instead of 64.
        float mx0 = -CUDART_INF_F, mx1 = mx0, mx2 = mx0, mx3 = mx0;
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          mx0 = max3(mx0, __uint_as_float(s0[c]), __uint_as_float(s0[c + 1]));
          mx1 = max3(mx1, __uint_as_float(s0[c + 2]), __uint_as_float(s0[c + 3]));
          mx2 = max3(mx2, __uint_as_float(s1[c]), __uint_as_float(s1[c + 1]));
          mx3 = max3(mx3, __uint_as_float(s1[c + 2]), __uint_as_float(s1[c + 3]));
        }
        mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        sh->half_max[buf][h][r] = mx;
      } else {
        sh->give_up = 1;
      }
      c_max += tick<kProf>() - tp;
      tp = tick<kProf>();
      softmax_pair_sync();
      c_sync += tick<kProf>() - tp;
      tp = tick<kProf>();
      if (sh->give_up) break;                 // uniform: every writer wrote before the barrier
      mx = fmaxf(mx, sh->half_max[buf][h ^ 1][r]);

      const float m_new = fmaxf(m_used, mx * mul);
      const bool grow = m_new > m_used + kRescaleThreshold;
      if (__any_sync(0xffffffffu, grow)) {
        const float factor = grow ? ex2_approx(m_used - m_new) : 1.0f;
        if (grow) m_used = m_new;
        l *= factor;
        if (jj > 0) {
          // O may still be receiving P V of the previous KV tile.  Its completion
          // is signalled on the barrier of that tile's parity, so a waiter that
          // skipped earlier phases is never more than one phase behind (a parity
          // wait cannot tell phases two apart).
          dead = !mbar_wait_warp(&sh->pv_done[(t - 1) & 1], ((t - 1) >> 1) & 1, abort, p.status,
                                 208);
          if (!dead) {
            tc_fence_after_sync();
            // Each half rescales its own 64 output columns.
            for (int c = h * 2; c < h * 2 + 2 && c < dv_chunks; ++c) {
              uint32_t o[32];
              tmem_ld_32x32(o_tmem + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
              tmem_st_32x32(o_tmem + c * 32, o);
            }
          }
        }
      }
      if (dead) continue;
      if (G::kPvFmt == Fmt::F16 && kHalfExp) {
        // fp16 P: the exponent x = S log2(e) - m is rounded to fp16 and two exponentials are
        // taken per special-function instruction (ex2.f16x2), whose packed result is the P
        // operand as it stands.  Rounding x costs P a relative error of ln 2 * |x| * 2^-11
        // (0.03 % at |x| = 1, 0.3 % at |x| = 8, where P itself is below 0.4 % of the row's
        // largest term), the same order as P's own rounding to fp16.  The row sum is taken from
        // the rounded values, eight pairs at a time in fp16 and then in fp32.
        uint32_t packed[32];
        float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
          uint32_t acc0 = 0u, acc1 = 0u;          // fp16 pair sums of this group (+0, +0)
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = g8 * 8 + u * 2;
            const uint32_t e0 = ex2_f16x2(pack_f16(fmaf(__uint_as_float(s0[c]), mul, -m_used),
                                                   fmaf(__uint_as_float(s0[c + 1]), mul, -m_used)));
            const uint32_t e1 = ex2_f16x2(pack_f16(fmaf(__uint_as_float(s1[c]), mul, -m_used),
                                                   fmaf(__uint_as_float(s1[c + 1]), mul, -m_used)));
            packed[c / 2] = e0;
            packed[16 + c / 2] = e1;
            acc0 = add_f16x2(acc0, e0);
            acc1 = add_f16x2(acc1, e1);
          }
          const uint32_t both = add_f16x2(acc0, acc1);
          sum0 += f16_lo(both);
          sum1 += f16_hi(both);
        }
        l += sum0 + sum1;
        c_exp += tick<kProf>() - tp;
        tp = tick<kProf>();
        tmem_st_32x32(s_tmem, packed);
      } else {
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float e0 = ex2_approx(fmaf(__uint_as_float(s0[c]), mul, -m_used));
        float e1 = ex2_approx(fmaf(__uint_as_float(s1[c]), mul, -m_used));
        sum0 += e0;
        sum1 += e1;
        s0[c] = __float_as_uint(e0);
        s1[c] = __float_as_uint(e1);
      }
      l += sum0 + sum1;
      c_exp += tick<kProf>() - tp;
      tp = tick<kProf>();
      if (!G::kPvHalf) {
        tmem_st_32x32(s_tmem, s0);
        tmem_st_32x32(s_tmem + 32, s1);
      } else {
        // Pack this half's 64 probabilities as 32 pairs of 16-bit values (bf16, or fp16 in the
        // mixed arm) over the start of its own S columns.
        uint32_t packed[32];
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          if (G::kPvFmt == Fmt::BF16) {
            packed[c] = pack_bf16(__uint_as_float(s0[2 * c]), __uint_as_float(s0[2 * c + 1]));
            packed[16 + c] = pack_bf16(__uint_as_float(s1[2 * c]), __uint_as_float(s1[2 * c + 1]));
          } else {
            packed[c] = pack_f16(__uint_as_float(s0[2 * c]), __uint_as_float(s0[2 * c + 1]));
            packed[16 + c] = pack_f16(__uint_as_float(s1[2 * c]), __uint_as_float(s1[2 * c + 1]));
          }
        }
        tmem_st_32x32(s_tmem, packed);
      }
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->p_full[buf]);
      c_store += tick<kProf>() - tp;
    }

    // ---- Q of the next piece, before this one's epilogue: every Q K^T of this piece has
    // completed (its S was read above), so Q's columns are free, and the MMA warp can run
    // the next piece's first Q K^T while O is being read out below.
    float next_row_mul = kLog2E32;
    {
      PieceCursor ahead = cursor;
      Piece nx;
      if (!dead && next_piece(p, ahead, nx)) {
        const int nb = nx.unit / p.q_tiles;
        next_row_mul = stage_q(nb, nx.unit - nb * p.q_tiles);
      }
    }

    // ---- epilogue: total row sum, normalise, store columns [64h, 64h+64) of O ----
    {
      const long long last = it + n_kv - 1;
      finish_piece(p, sh, o_tmem, h, r, row, b, whole, part_slot, l, m_used, dv_chunks,
                   &sh->pv_done[last & 1], static_cast<uint32_t>((last >> 1) & 1), dead);
    }
    if (sh->give_up) break;
    // The epilogue's reads of O are complete (tcgen05.wait::ld above): the next piece's first
    // P V may overwrite it.
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(&sh->o_free);
    it += n_kv;
    row_mul = next_row_mul;
    }  // pieces
    if (kProf && p.prof && quad == 0 && lane == 0 && h == 0) {
      p.prof[blockIdx.x * 16 + 7] = tick<kProf>() - t_start - wait_s;
      p.prof[blockIdx.x * 16 + 9] = c_load;
      p.prof[blockIdx.x * 16 + 10] = c_max;
      p.prof[blockIdx.x * 16 + 11] = c_sync;
      p.prof[blockIdx.x * 16 + 12] = c_exp;
      p.prof[blockIdx.x * 16 + 13] = c_store;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- helpers of the pipelined kernel: a row is shared by four threads, one per quarter -------------

// Q of one row tile for the pipelined kernel: this thread's 32 features [32 q4, 32 q4 + 32) of its
// row as 16 packed 16-bit pairs into tensor-memory columns [16 q4, 16 q4 + 16), then one arrival
// per warp on q_ready.  The fp16 arm stores the row over the power of two that brings its largest
// magnitude into [2^14, 2^15) (every thread reads the whole row for that: 128 features, from L2).
// Returns the factor that takes the row's S to exponent units, K's tile scale aside.

// Named barriers with separate arriving and waiting sides (ids 2 .. 5 in the pipelined kernel).
__device__ __forceinline__ void named_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// The kernel of the 16-bit arms (fp16 over powers of two, and bf16).  Same tiles and work split
// as above; 512 threads in six kinds of warps instead of three:
//   warp 0        K producer (one thread): K(t) through a ring of three 32 KB slots
//   warp 1        Q K^T issuer (one thread): S[t & 1] = Q K(t)^T, up to two tiles ahead of P V
//   warp 2        V producer (one thread): V^T(t) through a ring of three 32 KB slots of its own
//   warp 3        P V issuer (one thread): O += P(t) V(t)
//   warps 4-7     statistics: read S(t) first, keep every row's running maximum, rescale O when it
//                 grows by more than 2^8 and publish the reference maximum of the tile
//   warps 8-15    softmax: two warpgroups; warpgroup h takes the tiles at positions of parity h in
//                 this CTA's sequence, a warp all 128 columns of its 32 rows of such a tile
// Tensor memory: Q 0..63 | P 64..127 | S0 128..255 | S1 256..383 | O 384..511.  Packed Q takes 64
// columns, which leaves 64 for a buffer of P of its own: S[buf] is free again as soon as it has
// been *read* (s_free[buf]), not once P V has consumed the P written over it.
//
// Why this shape.  Measured on B200, with microbenchmarks and with builds of the kernel that leave
// parts out:
//   * the tensor pipe needs about 1140 - 1380 cycles per tile of 128 keys (16 MMAs of ~71 cycles
//     with A in tensor memory) -- the bound to reach; with the exponentials compiled out the
//     kernel runs at 1119 TFLOP/s on 8 heads of 16384 keys;
//   * a round trip of a warp to tensor memory (tcgen05.ld or st plus its wait) takes 400 - 700
//     cycles in the running kernel, and tcgen05.wait::ld waits for every load in flight, so loads
//     cannot be pipelined against arithmetic inside a warp.  A softmax warp that shares every tile
//     with three others (sixteen warps of 32 columns: the form this kernel had before) pays two
//     round trips per tile for a quarter of a row; a warp that takes whole rows of every other
//     tile pays them for four times the arithmetic, and the other warpgroup's exponentials run
//     meanwhile: 918 -> 972 TFLOP/s on 8 heads;
//   * the row maxima need all 128 columns of a row and sit in front of the exponentials; in the
//     statistics warps they are off the softmax warps' path, and because those warps see every
//     tile in order the two softmax warpgroups need nothing from each other;
//   * softmax warps wait for S(t) and its maximum on a named hardware barrier (bar.sync) rather
//     than by polling an mbarrier, so a waiting warp issues nothing (+5 to +8 %);
//   * Q K^T and P V are issued by two threads, K and V^T loaded by two, so that no stream waits
//     behind another's barrier in program order (one producer thread for both operands left the
//     Q K^T issuer waiting ~850 cycles a tile for K);
//   * two fp32 exponentials and one conversion of the pair beat ex2.approx.f16x2 on a converted
//     pair here (866 -> 918 in the sixteen-warp form), although the packed form was the faster
//     one in the 384-thread kernel above;
//   * Q of the next row block staged with one round of loads (each thread its own 64 columns, the
//     two halves of a row's largest magnitude meeting through shared memory) instead of nine
//     dependent rounds: 754 -> 829 TFLOP/s on one head of 16384, 972 -> 1015 on eight.
// setmaxnreg moves registers from the role and statistics warps to the softmax warps.
//
constexpr uint32_t kTmemP = 64;            // pipelined kernel: packed P, beside packed Q (0..63)

// Two fp32 operations in one instruction (sm_100 packed fp32): a pair is a 64-bit register.
__device__ __forceinline__ uint64_t f32x2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void f32x2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// Registers per thread after setmaxnreg.  setmaxnreg.inc blocks (without a limit) until the CTA's
// pool holds the registers it asks for, and the pool is only what this CTA's own warps gave back:
// the sum below must fit in what the CTA was launched with, kThreadsPipelined x the kernel's
// register count.  The host checks that count before every first launch on a device.
constexpr int kRegsRoles = 56, kRegsStats = 64, kRegsSoftmax = 192;
constexpr int kRegsAtLaunch = 128;            // what ptxas reports for __launch_bounds__(512, 1)
static_assert(128 * kRegsRoles + 128 * kRegsStats + 256 * kRegsSoftmax <= kThreadsPipelined * kRegsAtLaunch,
              "the softmax warps would wait for registers nobody releases");

template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// Q of one piece into tensor memory, by the eight softmax warps of the pipelined kernel: thread
// (h, r) loads columns 64 h .. 64 h + 63 of row r (sixteen 16-byte loads, all in flight at once;
// the producer has prefetched the rows into L2) and stores them packed to 16 bits.  On the fp16
// arm the two halves of a row's largest magnitude meet through shared memory and the 256-thread
// barrier, which every softmax warp must therefore reach: a warp that has given up (`idle`) comes
// here too and only skips the work.
template <Arm ARM>
__device__ __forceinline__ float stage_q_half(const Params& p, Shared* sh, uint32_t tmem_q, int head,
                                              int q_tile, int r, int h, int lane, int piece, bool idle) {
  using G = Geometry<ARM>;
  float row_mul = kLog2E32;
  const long long row = static_cast<long long>(q_tile) * kBQ + r;
  const float* qrow = p.q + (static_cast<size_t>(head) * p.nq + row) * p.d;
  const bool live = row < p.nq && !idle;
  const bool vec = (reinterpret_cast<uintptr_t>(p.q) & 15u) == 0 && p.d % 4 == 0;
  float qs = 1.0f;                             // a scale on the logits is a scale on Q
  if (p.logit_scale) {
    qs = __ldg(p.logit_scale);
    if (p.logit_divide) qs = 1.0f / qs;
  }
  float4 x[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const int col = h * 64 + 4 * e;
    x[e] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (live && vec && col + 4 <= p.d) {
      x[e] = *reinterpret_cast<const float4*>(qrow + col);
    } else if (live) {
      if (col + 0 < p.d) x[e].x = qrow[col + 0];
      if (col + 1 < p.d) x[e].y = qrow[col + 1];
      if (col + 2 < p.d) x[e].z = qrow[col + 2];
      if (col + 3 < p.d) x[e].w = qrow[col + 3];
    }
  }
#pragma unroll
  for (int e = 0; e < 16; ++e) { x[e].x *= qs; x[e].y *= qs; x[e].z *= qs; x[e].w *= qs; }
  float inv = 1.0f;
  if (G::kScaledQk) {
    float m = 0.0f;
#pragma unroll
    for (int e = 0; e < 16; ++e)
      m = fmaxf(m, fmaxf(fmaxf(fabsf(x[e].x), fabsf(x[e].y)), fmaxf(fabsf(x[e].z), fabsf(x[e].w))));
    sh->q_absmax[h][r] = m;
    softmax_pair_sync();
    m = fmaxf(sh->q_absmax[0][r], sh->q_absmax[1][r]);
    const float scale = f16_range_scale(m);
    inv = 1.0f / scale;
    row_mul = kLog2E32 * scale;
  }
  if (idle) return row_mul;
  uint32_t v[32];
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    if (G::kQkFmt == Fmt::F16) {
      v[2 * e + 0] = pack_f16(x[e].x * inv, x[e].y * inv);
      v[2 * e + 1] = pack_f16(x[e].z * inv, x[e].w * inv);
    } else {
      v[2 * e + 0] = pack_bf16(x[e].x, x[e].y);
      v[2 * e + 1] = pack_bf16(x[e].z, x[e].w);
    }
  }
  tmem_st_32x32(tmem_q + h * 32, v);
  // The statistics warps need the row's factor too (visible to them once q_ready has completed).
  if (h == 0) sh->row_mul[piece & 1][r] = row_mul;
  tmem_wait_st();
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(&sh->q_ready);
  return row_mul;
}

template <Arm ARM>
__global__ void __launch_bounds__(kThreadsPipelined, 1)
attention_pipelined_kernel(const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_vt, const Params p) {
  using G = Geometry<ARM>;
  static_assert(G::kQkHalf && G::kPvHalf, "the pipelined kernel is the one for 16-bit Q, K, P and V");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int kRing = 6;                   // six 32 KB slots in the space of three 64 KB ones
  constexpr int kSlotBytes = G::kSlotBytes;
  static_assert(kRing * kSlotBytes <= kRingBytes, "ring does not fit");
  uint8_t* ring = smem;
  Shared* sh = reinterpret_cast<Shared*>(ring + kRingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRing; ++s) mbar_init(&sh->kv_full[s], 1);
    mbar_init(&sh->q_ready, 8);            // one arrival per softmax warp
    mbar_init(&sh->o_free, 8);
    for (int u = 0; u < 4; ++u) {
      mbar_init(&sh->s_full[u], 1);
      mbar_init(&sh->pv_done[u], 1);
    }
    for (int u = 0; u < 2; ++u) {
      mbar_init(&sh->p_full[u], 4);        // the four warps of the softmax warpgroup that owns the tile
      mbar_init(&sh->s_free[u], 8);        // those four and the four statistics warps have read S
    }
    for (int u = 0; u < 4; ++u) {
      mbar_init(&sh->m_ready[u], 4);       // the four statistics warps (read at the end of a piece)
    }
    sh->abort.flag = 0;
    sh->give_up = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_slot, kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_slot;
  AbortState* abort = &sh->abort;
  trigger_dependent_launch();

  if (warp < 4) {
    setmaxnreg_dec<kRegsRoles>();
    // Three single-thread roles, one per warp, each walking the same sequence of pieces and key
    // tiles t = 0, 1, 2, ... of this CTA:
    //   warp 0  producer: K tile t into slot t % 3 of the K ring once Q K^T of tile t - 3 is done,
    //           then V^T tile t into slot t % 3 of the V ring once P V of tile t - 3 is
    //   warp 1  Q K^T issuer: S[t & 1] = Q K(t)^T once the softmax warps have read S of tile t - 2
    //   warp 3  P V issuer: O += P(t) V(t) once P(t) is in the P buffer
    // Two issuing threads instead of one keep the two streams independent: with one thread issuing
    // Q K^T(t + 2), P V(t), Q K^T(t + 3), ... in program order, a late P(t) (one warpgroup) held up
    // the Q K^T the other warpgroup was about to need.  The tensor pipe runs the instructions of
    // both threads in the order they reach it; every real dependence is a barrier wait.
    constexpr int kRingK = 3;
    const uint32_t ring_addr = smem_u32(ring);
    if (warp == 0 && lane == 0) {
      // K producer: K(t) into slot t % 3 of the K ring once Q K^T of tile t - 3 has completed.
      tma_prefetch_descriptor(&map_k);
      grid_dependency_wait();                 // K comes from the preparation kernel before this one
      const int d_chunks = (p.d + G::kQkChunkElems - 1) / G::kQkChunkElems;
      const bool q_prefetchable = (reinterpret_cast<uintptr_t>(p.q) & 15u) == 0;
      bool ok = true;
      int t = 0, slot = 0;                    // tile counter of this CTA; its slot in the ring
      long long waited = 0;
      PieceCursor cursor = pieces_begin(p);
      Piece pc;
      while (ok && next_piece(p, cursor, pc)) {
        const int b = pc.unit / p.q_tiles;
        {
          // Pull the Q rows of the piece after this one into L2 while this one runs.
          PieceCursor ahead = cursor;
          Piece nx;
          if (q_prefetchable && next_piece(p, ahead, nx) && nx.unit != pc.unit) {
            const int nb = nx.unit / p.q_tiles;
            const long long row0 = static_cast<long long>(nx.unit - nb * p.q_tiles) * kBQ;
            const long long rows = min(static_cast<long long>(kBQ), p.nq - row0);
            prefetch_l2_bulk(p.q + (static_cast<size_t>(nb) * p.nq + row0) * p.d,
                             static_cast<uint32_t>(rows * p.d * 4));
          }
        }
#pragma unroll 1
        for (int jj = 0; ok && jj < pc.n_kv; ++jj, ++t, slot = slot + 1 == kRingK ? 0 : slot + 1) {
          const int u = t - kRingK;
          // Slot reuse: Q K^T of tile t - 3 has completed.  The next completion on that barrier
          // is tile t + 1's, whose K this thread has not loaded yet, so the parity is unambiguous.
          if (t >= kRingK) {
            const long long t0 = tick<kProf>();
            ok = mbar_wait(&sh->s_full[u & 3], static_cast<uint32_t>((u >> 2) & 1), abort, p.status, 201);
            waited += tick<kProf>() - t0;
            if (!ok) break;
          }
          uint8_t* dst = ring + slot * kSlotBytes;
          mbar_arrive_expect_tx(&sh->kv_full[slot], d_chunks * kChunkBytes);
          for (int c = 0; c < d_chunks; ++c)
            tma_load_3d(dst + c * kChunkBytes, &map_k, &sh->kv_full[slot], c * G::kQkChunkElems,
                        (pc.kv_lo + jj) * kBKV, b);
        }
      }
      if (kProf && p.prof) p.prof[blockIdx.x * 16 + 0] = waited;
    } else if (warp == 2 && lane == 0) {
      // V producer: V^T(t) into slot t % 3 of the V ring once P V of tile t - 3 has completed.  A
      // thread of its own: P V runs about two tiles behind Q K^T, and behind one thread that
      // loads K(t) then V^T(t) the K loads waited with the V slots, and the Q K^T issuer for K.
      tma_prefetch_descriptor(&map_vt);
      grid_dependency_wait();                 // V^T comes from the preparation kernel before this one
      bool ok = true;
      int t = 0, slot = 0;
      PieceCursor cursor = pieces_begin(p);
      Piece pc;
      while (ok && next_piece(p, cursor, pc)) {
        const int b = pc.unit / p.q_tiles;
#pragma unroll 1
        for (int jj = 0; ok && jj < pc.n_kv; ++jj, ++t, slot = slot + 1 == kRingK ? 0 : slot + 1) {
          const int u = t - kRingK;
          if (t >= kRingK) {
            ok = mbar_wait(&sh->pv_done[u & 3], static_cast<uint32_t>((u >> 2) & 1), abort, p.status, 202);
            if (!ok) break;
          }
          uint8_t* dst = ring + (kRingK + slot) * kSlotBytes;
          mbar_arrive_expect_tx(&sh->kv_full[kRingK + slot], G::kPvTileChunks * kChunkBytes);
          for (int c = 0; c < G::kPvTileChunks; ++c)
            tma_load_3d(dst + c * kChunkBytes, &map_vt, &sh->kv_full[kRingK + slot],
                        (pc.kv_lo + jj) * kBKV + c * G::kPvChunkElems, 0, b);
        }
      }
    } else if (warp == 1 && lane == 0) {
      const uint32_t idesc_qk = make_idesc_fmt(G::kQkFmt, kBQ, kBKV);
      const int k_steps = (p.d + G::kQkStepElems - 1) / G::kQkStepElems;
      long long wait_k = 0, wait_q = 0, wait_f = 0, c_qk = 0;
      const long long t_start = tick<kProf>();
      bool ok = true;
      int t = 0, slot = 0;
      uint32_t phase = 0;                     // of the K ring's full barriers
      PieceCursor cursor = pieces_begin(p);
      Piece pc;
      for (int piece = 0; ok && next_piece(p, cursor, pc); ++piece) {
        // Q of this piece is in tensor memory.
        long long t0 = tick<kProf>();
        if (!(ok = mbar_wait(&sh->q_ready, piece & 1, abort, p.status, 203))) break;
        wait_q += tick<kProf>() - t0;
#pragma unroll 1
        for (int jj = 0; ok && jj < pc.n_kv; ++jj, ++t) {
          const int buf = t & 1;
          t0 = tick<kProf>();
          if (!(ok = mbar_wait(&sh->kv_full[slot], phase, abort, p.status, 204))) break;
          wait_k += tick<kProf>() - t0;
          t0 = tick<kProf>();
          // S[buf] was last used by tile t - 2; the softmax warps have it in registers once
          // s_free[buf] has completed for that tile.
          if (t >= 2 && !(ok = mbar_wait(&sh->s_free[buf], static_cast<uint32_t>(((t >> 1) - 1) & 1),
                                         abort, p.status, 211)))
            break;
          wait_f += tick<kProf>() - t0;
          tc_fence_after_sync();
          t0 = tick<kProf>();
          const uint64_t k_desc = make_smem_desc_sw128(ring_addr + slot * kSlotBytes);
          const uint32_t d_tmem = tmem_base + kTmemS + static_cast<uint32_t>(buf * kBKV);
          const uint32_t q_tmem = tmem_base + kTmemQ;
#pragma unroll
          for (int ks = 0; ks < G::kQkSteps; ++ks) {
            if (ks < k_steps)
              mma_ts<Kind::BF16>(d_tmem, q_tmem + ks * 8,
                                 k_desc + (((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4), idesc_qk,
                                 ks != 0 ? 1u : 0u);
          }
          mma_commit(&sh->s_full[t & 3]);        // S ready, and the K tile's slot is free
          c_qk += tick<kProf>() - t0;
          if (++slot == kRingK) { slot = 0; phase ^= 1u; }
        }
      }
      if (kProf && p.prof) {
        p.prof[blockIdx.x * 16 + 1] = wait_k;
        p.prof[blockIdx.x * 16 + 4] = tick<kProf>() - t_start;
        p.prof[blockIdx.x * 16 + 5] = wait_f;
        p.prof[blockIdx.x * 16 + 6] = c_qk;
        p.prof[blockIdx.x * 16 + 8] = wait_q;
      }
    } else if (warp == 3 && lane == 0) {
      const uint32_t n_pv = static_cast<uint32_t>((p.dv + 15) / 16 * 16);
      const uint32_t idesc_pv = make_idesc_fmt(G::kPvFmt, kBQ, n_pv);
      long long wait_v = 0, wait_p = 0, c_pv = 0;
      bool ok = true;
      int t = 0, slot = kRingK;
      uint32_t phase = 0;                     // of the V ring's full barriers
      PieceCursor cursor = pieces_begin(p);
      Piece pc;
      for (int piece = 0; ok && next_piece(p, cursor, pc); ++piece) {
#pragma unroll 1
        for (int jj = 0; ok && jj < pc.n_kv; ++jj, ++t) {
          long long t0 = tick<kProf>();
          if (!(ok = mbar_wait(&sh->kv_full[slot], phase, abort, p.status, 205))) break;
          // The first P V of a piece overwrites O: the piece before must have read it out.
          if (jj == 0 && piece > 0 &&
              !(ok = mbar_wait(&sh->o_free, static_cast<uint32_t>((piece - 1) & 1), abort, p.status, 210)))
            break;
          wait_v += tick<kProf>() - t0;
          t0 = tick<kProf>();
          if (!(ok = mbar_wait(&sh->p_full[t & 1], static_cast<uint32_t>((t >> 1) & 1), abort, p.status,
                               206)))
            break;
          wait_p += tick<kProf>() - t0;
          tc_fence_after_sync();
          t0 = tick<kProf>();
          const uint64_t v_desc = make_smem_desc_sw128(ring_addr + slot * kSlotBytes);
          const uint32_t d_tmem = tmem_base + kTmemO;
          const uint32_t p_tmem = tmem_base + kTmemP;
          if (jj == 0) {
            mma_ts<Kind::BF16>(d_tmem, p_tmem, v_desc, idesc_pv, 0u);
          } else {
            mma_ts<Kind::BF16>(d_tmem, p_tmem, v_desc, idesc_pv, 1u);
          }
#pragma unroll
          for (int ks = 1; ks < G::kPvSteps; ++ks)
            mma_ts<Kind::BF16>(d_tmem, p_tmem + ks * 8,
                               v_desc + (((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4), idesc_pv, 1u);
          mma_commit(&sh->pv_done[t & 3]);       // O updated; the V tile's slot and the P buffer are free
          c_pv += tick<kProf>() - t0;
          if (++slot == 2 * kRingK) { slot = kRingK; phase ^= 1u; }
        }
      }
      if (kProf && p.prof) {
        p.prof[blockIdx.x * 16 + 2] = wait_v;
        p.prof[blockIdx.x * 16 + 3] = wait_p;
        p.prof[blockIdx.x * 16 + 14] = c_pv;
      }
    }
  } else if (warp < 8) {
    // ---- statistics warpgroup: the reference maximum of every row after every key tile --------
    // Reads S(t) as soon as Q K^T has written it (16 columns at a time: this warpgroup gives its
    // registers to the softmax warps), keeps the running maximum of its 128 rows over the piece,
    // raises the reference when a tile exceeds it by more than 2^8, rescales O in that (rare) case,
    // and publishes the reference for the softmax warpgroup that owns the tile.  Because one
    // warpgroup sees every tile in order, the two softmax warpgroups need nothing from each other.
    // (Every lane waits on the barriers here: the one-lane-polls form of the wait made the
    // compiler ask for more than 96 registers in this branch, which the softmax warps need.)
    setmaxnreg_dec<kRegsStats>();
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t o_tmem = tmem_base + lane_bits + kTmemO;
    const int dv16 = (p.dv + 15) / 16;
    bool ok = true;
    int t = 0;
    PieceCursor cursor = pieces_begin(p);
    Piece pc;
    // On a failed wait this warp stops working but keeps arriving on the tiles' named barriers,
    // so that the softmax warps, which block on them, always get through (they then see the
    // abort flag and stop working too).
    for (int piece = 0; next_piece(p, cursor, pc); ++piece) {
      const int b = pc.unit / p.q_tiles;
      // The rows' Q scales of this piece are in shared memory once Q has been staged.
      if (ok) ok = mbar_wait(&sh->q_ready, piece & 1, abort, p.status, 215);
      const float row_mul = G::kScaledQk && ok ? sh->row_mul[piece & 1][r] : kLog2E32;
      float m_used = -CUDART_INF_F;
#pragma unroll 1
      for (int jj = 0; jj < pc.n_kv; ++jj, ++t) {
        if (ok) ok = mbar_wait(&sh->s_full[t & 3], static_cast<uint32_t>((t >> 2) & 1), abort, p.status, 216);
        if (ok) {
          tc_fence_after_sync();
          const uint32_t s_tmem = tmem_base + lane_bits + kTmemS + static_cast<uint32_t>((t & 1) * kBKV);
          const int col0 = (pc.kv_lo + jj) * kBKV;
          float mx = -CUDART_INF_F;
          float mul = row_mul;
          if (G::kScaledQk) mul *= __ldg(p.k_tile_scale + static_cast<size_t>(b) * p.kv_tiles + pc.kv_lo + jj);
          // One block of 32 columns at a time (this warpgroup runs on 64 registers).
#pragma unroll 1
          for (int c = 0; c < kBKV; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(s_tmem + c, v);
            tmem_wait_ld();
            if (col0 + c + 32 > p.nk) {
#pragma unroll
              for (int e = 0; e < 32; ++e)
                if (col0 + c + e >= p.nk) v[e] = __float_as_uint(-CUDART_INF_F);
            }
            float m0 = mx, m1 = -CUDART_INF_F, m2 = m1, m3 = m1;
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              m0 = max3(m0, __uint_as_float(v[e]), __uint_as_float(v[e + 1]));
              m1 = max3(m1, __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
              m2 = max3(m2, __uint_as_float(v[e + 4]), __uint_as_float(v[e + 5]));
              m3 = max3(m3, __uint_as_float(v[e + 6]), __uint_as_float(v[e + 7]));
            }
            mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
          }
          // S[t & 1] has been read here; the softmax warpgroup that owns the tile adds four arrivals.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh->s_free[t & 1]);
          const float m_new = fmaxf(m_used, mx * mul);
          const bool grow = m_new > m_used + kRescaleThreshold;
          if (jj > 0 && __any_sync(0xffffffffu, grow)) {
            // O holds the tiles up to t - 1 against the old reference once P V of tile t - 1 has
            // completed; P(t) is computed against the new one only after the publication below.
            ok = mbar_wait(&sh->pv_done[(t - 1) & 3], static_cast<uint32_t>(((t - 1) >> 2) & 1), abort,
                           p.status, 208);
            if (ok) {
              tc_fence_after_sync();
              const float factor = grow ? ex2_approx(m_used - m_new) : 1.0f;
#pragma unroll 1
              for (int c = 0; c < dv16; ++c) {
                uint32_t o[16];
                tmem_ld_32x16(o_tmem + c * 16, o);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
                tmem_st_32x16(o_tmem + c * 16, o);
              }
              tmem_wait_st();
              tc_fence_before_sync();
            }
          }
          if (grow) m_used = m_new;
          sh->pub_m[t & 3][r] = m_used;
        }
        // S(t) is ready and its reference maximum published: the softmax warps block on this
        // named barrier (one of four, by tile) instead of polling, so that while they wait they
        // issue nothing.
        named_arrive(2 + (t & 3), 128 + 128);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->m_ready[t & 3]);
      }
    }
  } else {
    // ---- softmax warpgroups: h = 0 takes the key tiles at even positions of this CTA's sequence,
    // h = 1 the odd ones; a warp holds all 128 columns of its 32 rows of a tile.  Per tile a warp
    // then makes two round trips to tensor memory (S in, P out) for twice the arithmetic of a
    // warp that shares every tile with three others.
    setmaxnreg_inc<kRegsSoftmax>();
    const int h = (warp - 8) >> 2;            // warpgroup: tiles of parity h; column half h of Q and O
    const int quad = warp & 3;                // TMEM lane quadrant
    const int r = quad * 32 + lane;           // row within the tile
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t o_tmem = tmem_base + lane_bits + kTmemO;
    const uint32_t p_tmem = tmem_base + lane_bits + kTmemP;
    const uint32_t tmem_q = tmem_base + lane_bits + kTmemQ;
    const int dv_chunks = (p.dv + 31) / 32;
    int it = 0;                               // key tiles of the pieces before this one
    long long wait_s = 0, c_a = 0, c_b = 0, c_exp = 0, c_tail = 0;   // kProf: cycles per phase
    const long long t_start = tick<kProf>();
    bool dead = false;                        // a wait gave up; keep hitting the barriers only
    float row_mul = kLog2E32;

    auto wait_bar = [&](uint64_t* bar, uint32_t parity, int code) {
      if (dead) return;
      dead = !mbar_wait_warp(bar, parity, abort, p.status, code);
      if (!dead) tc_fence_after_sync();
    };

    PieceCursor cursor = pieces_begin(p);
    Piece pc;
    int piece = 0;
    while (next_piece(p, cursor, pc)) {
      const int kv_lo = pc.kv_lo, n_kv = pc.n_kv;
      const int b = pc.unit / p.q_tiles;
      const int qt = pc.unit - b * p.q_tiles;
      const long long row = static_cast<long long>(qt) * kBQ + r;
      const bool whole = pc.whole;
      const int part_slot = 2 * static_cast<int>(blockIdx.x) + pc.ordinal;

      if (piece == 0) row_mul = stage_q_half<ARM>(p, sh, tmem_q, b, qt, r, h, lane, 0, false);

      // The piece after this one, whose Q is staged at the end of this one.
      float next_row_mul = kLog2E32;
      bool has_next = false;
      int next_b = 0, next_qt = 0;
      {
        PieceCursor ahead = cursor;
        Piece nx;
        if (next_piece(p, ahead, nx)) {
          has_next = true;
          next_b = nx.unit / p.q_tiles;
          next_qt = nx.unit - next_b * p.q_tiles;
        }
      }
      const int last = it + n_kv - 1;

      float m_mine = -CUDART_INF_F;           // the reference maximum l is expressed against
      float l = 0.0f;                         // row sum over this warpgroup's tiles
      float ks_ahead = 1.0f;                  // fp16 arm: K scale of this warpgroup's next tile
      bool have_scale = false;

#pragma unroll 1
      for (int jj = (it ^ h) & 1; jj < n_kv; jj += 2) {
        const int t = it + jj;
        uint32_t ra[32], rb[32], rc[32], rd[32];
        long long tp = tick<kProf>();
        {
          // S(t) has been written and read by the statistics warps, and its reference maximum is
          // in shared memory: they arrive on this barrier after both.  A warp that has given up
          // still comes here for every tile of its warpgroup, so nobody is left blocked.
          const long long t0 = tick<kProf>();
          named_sync(2 + (t & 3), 128 + 128);
          wait_s += tick<kProf>() - t0;
        }
        if (!dead && abort->flag) dead = true;
        if (dead) continue;
        tc_fence_after_sync();
        const uint32_t s_tmem = tmem_base + lane_bits + kTmemS + static_cast<uint32_t>((t & 1) * kBKV);
        tmem_ld_32x32(s_tmem, ra);
        tmem_ld_32x32(s_tmem + 32, rb);
        tmem_ld_32x32(s_tmem + 64, rc);
        tmem_ld_32x32(s_tmem + 96, rd);
        float mul = kLog2E32;
        if (G::kScaledQk) {
          const float* ks = p.k_tile_scale + static_cast<size_t>(b) * p.kv_tiles + kv_lo + jj;
          const float here = have_scale ? ks_ahead : __ldg(ks);
          have_scale = jj + 2 < n_kv;
          if (have_scale) ks_ahead = __ldg(ks + 2);
          mul = row_mul * here;
        }
        const float m_used = sh->pub_m[t & 3][r];
        if (m_mine != m_used) {
          l = m_mine == -CUDART_INF_F ? 0.0f : l * ex2_approx(m_mine - m_used);
          m_mine = m_used;
        }
        tmem_wait_ld();
        // S[t & 1] is in registers: with the statistics warps' arrivals, Q K^T of tile t + 2 may
        // overwrite it.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->s_free[t & 1]);
        c_a += tick<kProf>() - tp;
        tp = tick<kProf>();

        // Keys past the end of the sequence (last tile only).
        const int col0 = (kv_lo + jj) * kBKV;
        if (col0 + kBKV > p.nk) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (col0 + c >= p.nk) ra[c] = __float_as_uint(-CUDART_INF_F);
            if (col0 + 32 + c >= p.nk) rb[c] = __float_as_uint(-CUDART_INF_F);
            if (col0 + 64 + c >= p.nk) rc[c] = __float_as_uint(-CUDART_INF_F);
            if (col0 + 96 + c >= p.nk) rd[c] = __float_as_uint(-CUDART_INF_F);
          }
        }
        // 16 pairs of exponentials from `src` into dst[off .. off + 15], as a software pipeline.
        // The multiply-add in front of a pair of exponentials and the addition behind it are packed
        // fp32 instructions (two lanes each): five instructions per pair instead of seven.
        uint64_t sum2 = f32x2(0.0f, 0.0f);
        const uint64_t mul2 = f32x2(mul, mul), neg_m2 = f32x2(-m_used, -m_used);
        auto exp_block = [&](const uint32_t (&src)[32], uint32_t (&dst)[32], int off) {
          uint64_t x2[4];
          float ea[4], eb[4];
#pragma unroll
          for (int i = 0; i < 16 + 4; ++i) {
            if (i < 16)
              x2[i & 3] = fma_f32x2(f32x2(__uint_as_float(src[2 * i]), __uint_as_float(src[2 * i + 1])), mul2,
                                    neg_m2);
            if (i >= 1 && i - 1 < 16) {
              float fa, fb;
              f32x2_unpack(x2[(i - 1) & 3], fa, fb);
              ea[(i - 1) & 3] = ex2_approx(fa);
              eb[(i - 1) & 3] = ex2_approx(fb);
            }
            if (i >= 4) {
              const float y0 = ea[(i - 4) & 3], y1 = eb[(i - 4) & 3];
              dst[off + i - 4] = G::kPvFmt == Fmt::BF16 ? pack_bf16(y0, y1) : pack_f16(y0, y1);
              sum2 = add_f32x2(sum2, f32x2(y0, y1));
            }
          }
        };
        // The two halves of the tile run through the same 32 pairs of code in a loop that is not
        // unrolled (the second half's values are moved into the first half's registers), so that
        // what a softmax warp executes per tile stays short.
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          exp_block(ra, ra, 0);               // pair i lands in a register already consumed
          exp_block(rb, ra, 16);
          if (half == 0) {
            // P of keys 0 .. 63 moves to rd, the second half of S into ra and rb.
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              rb[c] = rd[c];
              rd[c] = ra[c];
              ra[c] = rc[c];
            }
          }
        }
        {
          float sum0, sum1;
          f32x2_unpack(sum2, sum0, sum1);
          l += sum0 + sum1;
        }
        c_exp += tick<kProf>() - tp;
        tp = tick<kProf>();
        // There is one P buffer for both warpgroups: it is free once P V of the tile before (the
        // other warpgroup's) has completed.
        if (jj > 0) {
          wait_bar(&sh->pv_done[(t - 1) & 3], static_cast<uint32_t>(((t - 1) >> 2) & 1), 212);
          if (dead) continue;
        }
        tmem_st_32x32(p_tmem, rd);            // keys 0 .. 63 of the tile
        tmem_st_32x32(p_tmem + 32, ra);       // keys 64 .. 127
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->p_full[t & 1]);
        c_tail += tick<kProf>() - tp;
      }

      // ---- end of the piece.  Both warpgroups need the final reference maximum, and Q's columns
      // may only be restaged once the last Q K^T has completed, which the warpgroup that did not
      // read that S has to wait for.
      float m_final = m_mine;
      if ((last & 1) != h) {
        wait_bar(&sh->s_full[last & 3], static_cast<uint32_t>((last >> 2) & 1), 214);
        wait_bar(&sh->m_ready[last & 3], static_cast<uint32_t>((last >> 2) & 1), 218);
        if (!dead) m_final = sh->pub_m[last & 3][r];
      }
      if (!dead && m_mine != m_final) l = m_mine == -CUDART_INF_F ? 0.0f : l * ex2_approx(m_mine - m_final);
      // Q of the next piece, before this one's epilogue, so that the Q K^T issuer can run the next
      // piece's first tiles while O is being read out below.  (The warpgroup that owns the last
      // tile has seen its S; the other one waited for it above.)
      if (has_next) next_row_mul = stage_q_half<ARM>(p, sh, tmem_q, next_b, next_qt, r, h, lane, piece + 1, dead);

      finish_piece(p, sh, o_tmem, h, r, row, b, whole, part_slot, l, m_final, dv_chunks,
                   &sh->pv_done[last & 3], static_cast<uint32_t>((last >> 2) & 1), dead);
      if (sh->give_up) break;
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->o_free);
      it += n_kv;
      row_mul = next_row_mul;
      ++piece;
    }  // pieces
    if (kProf && p.prof && quad == 0 && lane == 0 && h == 0) {
      p.prof[blockIdx.x * 16 + 7] = tick<kProf>() - t_start - wait_s;
      p.prof[blockIdx.x * 16 + 9] = c_a;
      p.prof[blockIdx.x * 16 + 10] = c_b;
      p.prof[blockIdx.x * 16 + 12] = c_exp;
      p.prof[blockIdx.x * 16 + 13] = c_tail;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Merges the pieces of every row tile that more than one CTA range touched:
// O = sum_s w_s O_s / sum_s w_s with w_s = l_s 2^(m_s - max m).  One CTA per row
// tile; which pieces exist follows from the same range arithmetic the main
// kernel uses.
struct CombineArgs {
  const float* part_o;
  const float* part_m;
  const float* part_l;
  float* o;
  int nq, dv, q_tiles, kv_tiles, ctas;   // kv_tiles: granules per row tile (Params::kv_coarse)
  int first_tail_unit;     // row tiles before it were taken whole
  long long iters_base;    // the tail's flat (row tile, granule) sequence, cut as in the main kernel
  int iters_rem;
};

__device__ __forceinline__ long long range_start(const CombineArgs& a, int g) {
  return g * a.iters_base + min(g, a.iters_rem);
}

__device__ __forceinline__ int cta_of(const CombineArgs& a, long long it) {
  const long long fat = static_cast<long long>(a.iters_rem) * (a.iters_base + 1);
  if (it < fat) return static_cast<int>(it / (a.iters_base + 1));
  return a.iters_rem + static_cast<int>((it - fat) / max(a.iters_base, 1ll));
}

__global__ void __launch_bounds__(256)
attention_combine_kernel(const CombineArgs a) {
  constexpr int kRowsPerCta = 16;
  grid_dependency_wait();                   // every CTA, before any exit: the pieces come from the
                                            // attention kernel this one may have been launched under
  const int tail_unit = blockIdx.x / (kBQ / kRowsPerCta);
  const int row0 = (blockIdx.x % (kBQ / kRowsPerCta)) * kRowsPerCta;
  const int unit = a.first_tail_unit + tail_unit;
  const long long lo = static_cast<long long>(tail_unit) * a.kv_tiles, hi = lo + a.kv_tiles;
  const int g_first = cta_of(a, lo), g_last = cta_of(a, hi - 1);
  if (g_first == g_last) return;            // one CTA covered the whole tile and stored O itself
  const int b = unit / a.q_tiles, qt = unit - b * a.q_tiles;
  const int dv4 = (a.dv + 3) / 4;
  const bool vec = a.dv % 4 == 0 && (reinterpret_cast<uintptr_t>(a.o) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(a.part_o) & 15u) == 0;
  // A row tile is cut into at most kMaxPieces pieces when every CTA has at least half a row tile
  // of work (the usual case); then a thread issues every load of its item at once instead of one
  // dependent round trip to L2 per piece and quantity.
  constexpr int kMaxPieces = 4;
  const int pieces = g_last - g_first + 1;
  int slots[kMaxPieces];
#pragma unroll
  for (int k = 0; k < kMaxPieces; ++k) {
    const int g = min(g_first + k, g_last);
    slots[k] = 2 * g + (range_start(a, g) >= lo ? 0 : 1);
  }
  for (int i = threadIdx.x; i < kRowsPerCta * dv4; i += 256) {
    const int r = row0 + i / dv4, c = (i % dv4) * 4;
    const long long row = static_cast<long long>(qt) * kBQ + r;
    if (row >= a.nq) continue;
    float* dst = a.o + (static_cast<size_t>(b) * a.nq + row) * a.dv + c;
    if (vec && pieces <= kMaxPieces) {
      float pm[kMaxPieces], pl[kMaxPieces];
      float4 po[kMaxPieces];
#pragma unroll
      for (int k = 0; k < kMaxPieces; ++k) {
        const size_t prow = static_cast<size_t>(slots[k]) * kBQ + r;
        const bool live = k < pieces;
        pm[k] = live ? a.part_m[prow] : -CUDART_INF_F;
        pl[k] = live ? a.part_l[prow] : 0.0f;
        po[k] = live ? *reinterpret_cast<const float4*>(a.part_o + prow * a.dv + c)
                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
      float m = pm[0];
#pragma unroll
      for (int k = 1; k < kMaxPieces; ++k) m = fmaxf(m, pm[k]);
      float wsum = 0.0f;
      float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int k = 0; k < kMaxPieces; ++k) {
        const float w = k < pieces ? pl[k] * exp2f(pm[k] - m) : 0.0f;
        wsum += w;
        acc.x += w * po[k].x; acc.y += w * po[k].y; acc.z += w * po[k].z; acc.w += w * po[k].w;
      }
      const float inv = 1.0f / wsum;
      *reinterpret_cast<float4*>(dst) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
      continue;
    }
    float m = -CUDART_INF_F;
    for (int g = g_first; g <= g_last; ++g) {
      const int slot = 2 * g + (range_start(a, g) >= lo ? 0 : 1);
      m = fmaxf(m, a.part_m[static_cast<size_t>(slot) * kBQ + r]);
    }
    float wsum = 0.0f;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int g = g_first; g <= g_last; ++g) {
      const int slot = 2 * g + (range_start(a, g) >= lo ? 0 : 1);
      const size_t prow = static_cast<size_t>(slot) * kBQ + r;
      const float w = a.part_l[prow] * exp2f(a.part_m[prow] - m);
      wsum += w;
      const float* src = a.part_o + prow * a.dv + c;
      if (vec) {
        const float4 v = *reinterpret_cast<const float4*>(src);
        acc[0] += w * v.x; acc[1] += w * v.y; acc[2] += w * v.z; acc[3] += w * v.w;
      } else {
        for (int e = 0; e < 4 && c + e < a.dv; ++e) acc[e] += w * src[e];
      }
    }
    const float inv = 1.0f / wsum;
    if (vec) {
      *reinterpret_cast<float4*>(dst) = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
    } else {
      for (int e = 0; e < 4 && c + e < a.dv; ++e) dst[e] = acc[e] * inv;
    }
  }
}

// Debugging aid: when set (device pointer to 16 counters per CTA), the kernel
// records how many cycles each role spent waiting on its barriers.
unsigned long long* g_attention_profile = nullptr;

// Number of CTAs for a call: one per SM, fewer when there is too little work to
// give each at least two key tiles, or one granule at which a row tile's keys may be divided.
int choose_ctas(long long units, long long kv_tiles, long long kv_coarse, int sms) {
  if (units >= sms) return sms;
  long long g = units * kv_tiles / 2;
  if (g > units * kv_coarse) g = units * kv_coarse;
  if (g < 1) g = 1;
  if (g > sms) g = sms;
  return static_cast<int>(g);
}

// Key tiles per granule for a caller's granule in keys (0 = one tile; never more than a row's).
long long granule_tiles(size_t kv_granule, long long kv_tiles) {
  long long t = kv_granule == 0 ? 1 : static_cast<long long>((kv_granule - 1) / kBKV + 1);
  if (kv_granule > static_cast<size_t>(kv_tiles) * kBKV) t = kv_tiles;
  return t < 1 ? 1 : (t > kv_tiles ? kv_tiles : t);
}

// SMs the persistent kernel leaves free (for a communication kernel running next to it).
std::atomic<int> g_reserved_sms{0};

// I_B200_DEPENDENT_LAUNCH=0 launches the kernels of a call strictly one after another.
const bool g_dependent_launch = [] {
  const char* v = std::getenv("I_B200_DEPENDENT_LAUNCH");
  return !(v && v[0] == '0');
}();

int device_sms() {
  int sms = kNumSMs;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int reserved = g_reserved_sms.load();
  return sms - reserved > 8 ? sms - reserved : 8;
}

}  // namespace

void set_attention_profile(unsigned long long* p) { g_attention_profile = p; }
void set_reserved_sms(int n) { g_reserved_sms.store(n < 0 ? 0 : n); }
int reserved_sms() { return g_reserved_sms.load(); }

size_t attention_tcgen05_partial_floats(size_t batch, size_t nq, size_t nk, size_t dv, int* ctas_out) {
  const long long units = static_cast<long long>((nq + kBQ - 1) / kBQ) * static_cast<long long>(batch);
  const long long kv_tiles = static_cast<long long>((nk + kBKV - 1) / kBKV);
  // The finest division (one key tile) gives the most CTAs: the size below serves every granule.
  const int ctas = choose_ctas(units, kv_tiles, kv_tiles, device_sms());
  if (ctas_out) *ctas_out = ctas;
  // Two pieces per CTA (the ends of its range), 128 rows each, O plus (m, l).
  return static_cast<size_t>(2) * ctas * kBQ * (dv + 2);
}

int attention_tcgen05(const float* q, const void* k, const void* vt, float* o, size_t batch,
                      size_t nq, size_t nk, size_t d, size_t dv, size_t d_pitch, size_t nk_pitch,
                      AttentionArm arm, const float* v_scale, const float* k_tile_scale,
                      const float* logit_scale, bool logit_divide, bool follows_prepare,
                      float* partials, size_t kv_granule, cudaStream_t s) {
  const bool f16 = arm == AttentionArm::F16;
  const bool bf16 = arm == AttentionArm::BF16 || f16;      // K is 16-bit
  const bool mixed = arm == AttentionArm::MIXED || f16;    // V^T is fp16 over per-head scales
  if (f16 && (!k_tile_scale || !v_scale)) return fail("ib_attention: the fp16 arm needs its scales");
  if (batch == 0 || nq == 0) return 0;
  if (nk == 0) return fail("ib_attention: no keys");
  if (nq >= (1u << 30) || nk >= (1u << 30) || batch >= (1u << 20))
    return fail("ib_attention: shape too large");
  if (d % 4 != 0 || d < 4 || d > 128 || dv < 1 || dv > 128)
    return fail("ib_attention: head dimensions outside the fused kernel's range");
  const int smem_bytes = 1024 + kRingBytes + static_cast<int>(sizeof(Shared)) + 64;
  // The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of each kernel.
  {
    static OncePerDevice configured;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail("ib_attention: cannot identify the current device");
    const int rc = configured.run(dev, [smem_bytes] {
      cudaError_t err = cudaSuccess;
      const void* variants[] = {reinterpret_cast<const void*>(&attention_tf32_kernel<Arm::TF32>),
                                reinterpret_cast<const void*>(&attention_tf32_kernel<Arm::MIXED>),
                                reinterpret_cast<const void*>(&attention_pipelined_kernel<Arm::BF16>),
                                reinterpret_cast<const void*>(&attention_pipelined_kernel<Arm::F16>)};
      for (const void* fn : variants)
        if (err == cudaSuccess)
          err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
      // The pipelined kernels redistribute registers between their warpgroups; see kRegsAtLaunch.
      for (int v = 2; v < 4 && err == cudaSuccess; ++v) {
        cudaFuncAttributes attr{};
        err = cudaFuncGetAttributes(&attr, variants[v]);
        if (err == cudaSuccess && attr.numRegs < kRegsAtLaunch)
          return fail("ib_attention: the pipelined kernel was built with " + std::to_string(attr.numRegs) +
                      " registers per thread, fewer than its register redistribution assumes");
      }
      if (err != cudaSuccess)
        return fail(std::string("ib_attention: cannot reserve shared memory: ") +
                    cudaGetErrorString(err));
      return 0;
    });
    if (rc == -2) return fail("ib_attention: cannot identify the current device");
    if (rc != 0) return rc;
  }
  Params p{};
  p.q = q;
  p.nq = static_cast<int>(nq);
  p.nk = static_cast<int>(nk);
  p.d = static_cast<int>(d);
  p.dv = static_cast<int>(dv);
  p.batch = static_cast<int>(batch);
  p.q_tiles = static_cast<int>((nq + kBQ - 1) / kBQ);
  p.kv_tiles = static_cast<int>((nk + kBKV - 1) / kBKV);
  if (!partials) return fail("ib_attention: workspace for partial results is missing");
  const long long units = static_cast<long long>(p.q_tiles) * p.batch;
  // Where a row tile's key range may be cut between CTAs: at multiples of the caller's granule
  // (whole 128-key tiles); a granule of the whole range or more means never.
  p.coarse = static_cast<int>(granule_tiles(kv_granule, p.kv_tiles));
  p.kv_coarse = (p.kv_tiles + p.coarse - 1) / p.coarse;
  const int ctas = choose_ctas(units, p.kv_tiles, p.kv_coarse, device_sms());
  p.ctas = ctas;
  p.full_waves = static_cast<int>(units / ctas);
  const long long tail_units = units - static_cast<long long>(p.full_waves) * ctas;
  const long long tail_iters = tail_units * p.kv_coarse;
  p.iters_base = tail_iters / ctas;
  p.iters_rem = static_cast<int>(tail_iters % ctas);
  p.o = o;
  p.v_scale = mixed ? v_scale : nullptr;
  p.k_tile_scale = f16 ? k_tile_scale : nullptr;
  p.logit_scale = logit_scale;
  p.logit_divide = logit_divide ? 1 : 0;
  const size_t slots_rows = static_cast<size_t>(2) * ctas * kBQ;
  p.part_o = partials;
  p.part_m = partials + slots_rows * dv;
  p.part_l = p.part_m + slots_rows;
  p.status = device_status_word(s);
  if (!p.status) return fail("ib_attention: cannot allocate the device status word");
  p.prof = g_attention_profile;

  // K: fp32 (TF32-rounded) unless the whole call is bf16; V^T: fp32 only in the pure TF32 arm
  // (the 16-bit tensor map serves fp16 as well as bf16: TMA moves the bytes and fills zeros).
  const size_t k_pitch = bf16 ? d_pitch : d;
  CUtensorMap map_k, map_vt;
  if (bf16) {
    if (int rc = make_tensor_map_bf16(&map_k, k, batch, nk, d, k_pitch, nk * k_pitch, kBKV)) return rc;
  } else {
    if (int rc = make_tensor_map_f32(&map_k, static_cast<const float*>(k), batch, nk, d, k_pitch,
                                     nk * k_pitch, kBKV))
      return rc;
  }
  if (bf16 || mixed) {
    if (int rc = make_tensor_map_bf16(&map_vt, vt, batch, dv, nk, nk_pitch, dv * nk_pitch, 128))
      return rc;
  } else {
    if (int rc = make_tensor_map_f32(&map_vt, static_cast<const float*>(vt), batch, dv, nk, nk_pitch,
                                     dv * nk_pitch, 128))
      return rc;
  }

  // Both launches carry the programmatic-serialization attribute: the attention
  // kernel's set-up and its Q load run under the tail of the preparation kernel,
  // and the merge kernel's launch latency under the attention kernel.  The
  // attention kernel reads Q before it waits for its predecessor, so it only gets
  // the attribute when that predecessor is this library's preparation kernel.
  cudaLaunchAttribute overlap{};
  overlap.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  overlap.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas));
  cfg.blockDim = dim3(f16 || bf16 ? kThreadsPipelined : kThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = s;
  cfg.attrs = &overlap;
  cfg.numAttrs = g_dependent_launch && follows_prepare ? 1 : 0;
  cudaError_t launched;
  if (f16)
    launched = cudaLaunchKernelEx(&cfg, attention_pipelined_kernel<Arm::F16>, map_k, map_vt, p);
  else if (bf16)
    launched = cudaLaunchKernelEx(&cfg, attention_pipelined_kernel<Arm::BF16>, map_k, map_vt, p);
  else if (mixed)
    launched = cudaLaunchKernelEx(&cfg, attention_tf32_kernel<Arm::MIXED>, map_k, map_vt, p);
  else
    launched = cudaLaunchKernelEx(&cfg, attention_tf32_kernel<Arm::TF32>, map_k, map_vt, p);
  if (launched != cudaSuccess)
    return fail(std::string("ib_attention (tcgen05): launch failed: ") + cudaGetErrorString(launched));
  count_launch();
  // Tail row tiles shared by several CTA ranges exist unless the ranges fall on tile boundaries.
  if (tail_units > 0 && !(p.iters_rem == 0 && p.iters_base % p.kv_coarse == 0)) {
    CombineArgs a{p.part_o, p.part_m, p.part_l, o, p.nq, p.dv, p.q_tiles, p.kv_coarse, ctas,
                  p.full_waves * ctas, p.iters_base, p.iters_rem};
    cfg.numAttrs = g_dependent_launch ? 1 : 0;
    cfg.gridDim = dim3(static_cast<unsigned>(tail_units * 8));
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    launched = cudaLaunchKernelEx(&cfg, attention_combine_kernel, a);
    if (launched != cudaSuccess)
      return fail(std::string("ib_attention (combine): launch failed: ") + cudaGetErrorString(launched));
    count_launch();
  }
  return 0;
}

}  // namespace ib

#if IB_ATTN_PROFILE
// Development builds only (-DIB_ATTN_PROFILE=1): device pointer to 16 counters per CTA.
extern "C" void ib_debug_set_attention_profile(unsigned long long* device_counters) {
  ib::set_attention_profile(device_counters);
}
#endif
