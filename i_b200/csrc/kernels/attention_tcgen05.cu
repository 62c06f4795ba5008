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

#include "common.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace ib {
namespace {

using namespace sm100;

constexpr int kBQ = 128;           // query rows per CTA
constexpr int kBKV = 128;          // keys per KV tile
constexpr int kThreads = 384;
constexpr int kChunkBytes = 128 * 128;     // 128 rows of 128 bytes: 32 fp32 or 64 bf16 per row
constexpr int kMaxRing = 3;

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
  long long iters_base;   // tail (row tile, key tile) pairs per CTA: CTA g takes iters_base, plus
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
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t pv_done[2];       // [KV tile parity]: see the note at its wait
  uint32_t tmem_slot;
  AbortState abort;
  int give_up;               // raised before a named barrier, read after it
  float half_max[2][2][kBQ]; // [iteration parity][warpgroup][row]
  float half_sum[2][kBQ];
};

// One contiguous run of key tiles of one row tile.
struct Piece {
  int unit;        // row tile index over the whole call (head * q_tiles + tile)
  int kv_lo, n_kv;
  bool whole;      // covers every key tile: the result is final
  int ordinal;     // 0 = first tail piece of this CTA, 1 = a later one
};

struct PieceCursor {
  int wave;
  long long lo, cur, hi;
};

__device__ __forceinline__ PieceCursor pieces_begin(const Params& p) {
  PieceCursor c;
  const int g = static_cast<int>(blockIdx.x);
  c.wave = 0;
  c.lo = g * p.iters_base + min(g, p.iters_rem);
  c.hi = c.lo + p.iters_base + (g < p.iters_rem ? 1 : 0);
  c.cur = c.lo;
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
  if (c.cur >= c.hi) return false;
  const int tail_unit = static_cast<int>(c.cur / p.kv_tiles);
  out.unit = p.full_waves * p.ctas + tail_unit;
  out.kv_lo = static_cast<int>(c.cur - static_cast<long long>(tail_unit) * p.kv_tiles);
  out.n_kv = static_cast<int>(min(static_cast<long long>(p.kv_tiles - out.kv_lo), c.hi - c.cur));
  out.whole = out.kv_lo == 0 && out.n_kv == p.kv_tiles;
  out.ordinal = c.cur == c.lo ? 0 : 1;
  c.cur += out.n_kv;
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

template <bool PROF>
__device__ __forceinline__ long long tick() {
  return PROF ? clock64() : 0ll;
}

__device__ __forceinline__ void softmax_pair_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

// PROF = true compiles in the cycle counters written to Params::prof.
template <bool PROF, Arm ARM>
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
    if (lane == 0) {
      tma_prefetch_descriptor(&map_k);
      tma_prefetch_descriptor(&map_vt);
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
      // meets every event once and in order, and with three slots the next-but-one
      // event on the same barrier needs a tile this producer has not loaded yet, so
      // a parity wait is never two phases behind (a deeper ring would break that).
      uint64_t* occupant_bar[kRing] = {};
      uint32_t occupant_parity[kRing] = {};
      long long tile_k = 0, tile_v = 0;       // tile counters of the next K / V load
      auto acquire = [&](int code) {
        if (!occupant_bar[slot]) return;
        const long long t0 = tick<PROF>();
        ok = mbar_wait(occupant_bar[slot], occupant_parity[slot], abort, p.status, code);
        waited += tick<PROF>() - t0;
      };
      auto load_k = [&](int j) {
        acquire(201);
        if (!ok) return;
        uint8_t* dst = ring + slot * kSlotBytes;
        mbar_arrive_expect_tx(&sh->kv_full[slot], d_chunks * kChunkBytes);
        for (int c = 0; c < d_chunks; ++c)
          tma_load_3d(dst + c * kChunkBytes, &map_k, &sh->kv_full[slot], c * G::kQkChunkElems,
                      j * kBKV, b);
        occupant_bar[slot] = &sh->s_full[tile_k & 1];
        occupant_parity[slot] = static_cast<uint32_t>((tile_k >> 1) & 1);
        ++tile_k;
        if (++slot == kRing) slot = 0;
      };
      auto load_v = [&](int j) {
        acquire(202);
        if (!ok) return;
        uint8_t* dst = ring + slot * kSlotBytes;
        mbar_arrive_expect_tx(&sh->kv_full[slot], G::kPvTileChunks * kChunkBytes);
        for (int c = 0; c < G::kPvTileChunks; ++c)
          tma_load_3d(dst + c * kChunkBytes, &map_vt, &sh->kv_full[slot],
                      j * kBKV + c * G::kPvChunkElems, 0, b);
        occupant_bar[slot] = &sh->pv_done[tile_v & 1];
        occupant_parity[slot] = static_cast<uint32_t>((tile_v >> 1) & 1);
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
        load_k(pc.kv_lo);
        for (int jj = 0; ok && jj < pc.n_kv; ++jj) {
          if (jj + 1 < pc.n_kv) load_k(pc.kv_lo + jj + 1);
          if (ok) load_v(pc.kv_lo + jj);
        }
      }
      if (PROF && p.prof) p.prof[blockIdx.x * 16 + 0] = waited;
    }
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
      const long long t_start = tick<PROF>();
      bool ok = true;
      long long it = 0;                       // key tiles issued so far by this CTA

      // S[buf] = Q K^T from the K tile in the current slot (A = Q in tensor memory).
      auto issue_qk = [&](int buf) {
        const long long t0 = tick<PROF>();
        if (!(ok = mbar_wait(&sh->kv_full[slot], phase, abort, p.status, 204))) return;
        wait_k += tick<PROF>() - t0;
        tc_fence_after_sync();
        // One descriptor per slot; a K step moves it by a compile-time constant
        // (32 bytes inside the swizzled row, 16 KB to the next 32-feature chunk),
        // so the issuing thread spends one 64-bit add per MMA.
        const long long ti = tick<PROF>();
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
        issue_qk_cycles += tick<PROF>() - ti;
        if (++slot == kRing) { slot = 0; phase ^= 1; }
      };
      // O += P[buf] V from the V^T tile in the current slot (A = P in tensor memory).
      auto issue_pv = [&](long long t, bool first_of_piece, int piece) {
        const int buf = static_cast<int>(t & 1);
        long long t0 = tick<PROF>();
        if (!(ok = mbar_wait(&sh->kv_full[slot], phase, abort, p.status, 205))) return;
        // The first P V of a piece overwrites O: the piece before must have read it out.
        if (first_of_piece && piece > 0 &&
            !(ok = mbar_wait(&sh->o_free, static_cast<uint32_t>((piece - 1) & 1), abort, p.status, 210)))
          return;
        wait_v += tick<PROF>() - t0;
        t0 = tick<PROF>();
        if (!(ok = mbar_wait(&sh->p_full[buf], (t >> 1) & 1, abort, p.status, 206))) return;
        wait_p += tick<PROF>() - t0;
        tc_fence_after_sync();
        const long long ti = tick<PROF>();
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
        issue_pv_cycles += tick<PROF>() - ti;
        if (++slot == kRing) { slot = 0; phase ^= 1; }
      };

      PieceCursor cursor = pieces_begin(p);
      Piece pc;
      for (int piece = 0; ok && next_piece(p, cursor, pc); ++piece) {
        const int n_kv = pc.n_kv;
        // Q of this piece is in tensor memory.
        const long long tq = tick<PROF>();
        if (!(ok = mbar_wait(&sh->q_ready, piece & 1, abort, p.status, 203))) break;
        wait_q += tick<PROF>() - tq;
        tc_fence_after_sync();
        issue_qk(static_cast<int>(it & 1));
        for (int jj = 0; ok && jj < n_kv; ++jj) {
          if (jj + 1 < n_kv) issue_qk(static_cast<int>((it + jj + 1) & 1));
          if (ok) issue_pv(it + jj, jj == 0, piece);
        }
        it += n_kv;
      }
      if (PROF && p.prof) {
        p.prof[blockIdx.x * 16 + 1] = wait_k;
        p.prof[blockIdx.x * 16 + 2] = wait_v;
        p.prof[blockIdx.x * 16 + 5] = issue_qk_cycles;
        p.prof[blockIdx.x * 16 + 6] = issue_pv_cycles;
        p.prof[blockIdx.x * 16 + 3] = wait_p;
        p.prof[blockIdx.x * 16 + 4] = tick<PROF>() - t_start;
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
    const long long t_start = tick<PROF>();
    bool dead = false;                        // a wait gave up; keep hitting the barriers only
    float row_mul = kLog2E32;                 // S of this thread's row -> exponent units (see stage_q)

    // Q of one row tile: global -> operand type (nearest) -> tensor memory, this thread's 64
    // features [64h, 64h+64) of its row; then one arrival per warp on q_ready.
    // Returns the factor that takes this row's S to the exponent's units, K's tile scale aside:
    // log2(e), times the row's own power of two where Q is stored scaled.
    auto stage_q = [&](int head, int q_tile) -> float {
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
      if (!G::kQkHalf) {
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
          tmem_st_32x32(tmem_base + lane_bits + kTmemQ + col0, v);
        }
      } else {
        // 16-bit pairs, two features per column: features [64h, 64h+64) -> columns [32h, 32h+32).
        // The whole row's largest magnitude decides the power of two that brings the row into
        // [2^14, 2^15); the other half of the row is read for that alone (once per row tile,
        // from L2, eight loads at a time), then this thread's own 64 features, all in flight
        // together.
        float m = 0.0f;
        if (G::kScaledQk) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            float4 other[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) other[e] = load4((h ^ 1) * 64 + half * 32 + 4 * e);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              m = fmaxf(m, fmaxf(fmaxf(fabsf(other[e].x), fabsf(other[e].y)),
                                 fmaxf(fabsf(other[e].z), fabsf(other[e].w))));
          }
        }
        float4 own[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) own[e] = load4(h * 64 + 4 * e);
        float inv = 1.0f;
        if (G::kScaledQk) {
#pragma unroll
          for (int e = 0; e < 16; ++e)
            m = fmaxf(m, fmaxf(fmaxf(fabsf(own[e].x), fabsf(own[e].y)),
                               fmaxf(fabsf(own[e].z), fabsf(own[e].w))));
          const float scale = f16_range_scale(m);
          inv = 1.0f / scale;
          row_mul = kLog2E32 * scale;
        }
        uint32_t v[32];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float4 x = own[e];
          if (G::kQkFmt == Fmt::F16) {
            v[2 * e + 0] = pack_f16(x.x * inv, x.y * inv);
            v[2 * e + 1] = pack_f16(x.z * inv, x.w * inv);
          } else {
            v[2 * e + 0] = pack_bf16(x.x, x.y);
            v[2 * e + 1] = pack_bf16(x.z, x.w);
          }
        }
        tmem_st_32x32(tmem_base + lane_bits + kTmemQ + h * 32, v);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->q_ready);
      return row_mul;
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
        const long long t0 = tick<PROF>();
        dead = !mbar_wait_warp(&sh->s_full[buf], (t >> 1) & 1, abort, p.status, 207);
        wait_s += tick<PROF>() - t0;
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
      long long tp = tick<PROF>();
      if (!dead) {
        tc_fence_after_sync();
        tmem_ld_32x32(s_tmem, s0);
        tmem_ld_32x32(s_tmem + 32, s1);
        tmem_wait_ld();
        c_load += tick<PROF>() - tp;
        tp = tick<PROF>();
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
      c_max += tick<PROF>() - tp;
      tp = tick<PROF>();
      softmax_pair_sync();
      c_sync += tick<PROF>() - tp;
      tp = tick<PROF>();
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
        c_exp += tick<PROF>() - tp;
        tp = tick<PROF>();
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
      c_exp += tick<PROF>() - tp;
      tp = tick<PROF>();
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
      c_store += tick<PROF>() - tp;
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
    if (!sh->give_up && !dead) {
      const long long last = it + n_kv - 1;
      dead = !mbar_wait_warp(&sh->pv_done[last & 1], (last >> 1) & 1, abort, p.status, 209);
    }
    sh->half_sum[h][r] = l;
    if (dead) sh->give_up = 1;
    softmax_pair_sync();
    if (!sh->give_up) {
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
    if (sh->give_up) break;
    // The epilogue's reads of O are complete (tcgen05.wait::ld above): the next piece's first
    // P V may overwrite it.
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(&sh->o_free);
    it += n_kv;
    row_mul = next_row_mul;
    }  // pieces
    if (PROF && p.prof && quad == 0 && lane == 0 && h == 0) {
      p.prof[blockIdx.x * 16 + 7] = tick<PROF>() - t_start - wait_s;
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

// Merges the pieces of every row tile that more than one CTA range touched:
// O = sum_s w_s O_s / sum_s w_s with w_s = l_s 2^(m_s - max m).  One CTA per row
// tile; which pieces exist follows from the same range arithmetic the main
// kernel uses.
struct CombineArgs {
  const float* part_o;
  const float* part_m;
  const float* part_l;
  float* o;
  int nq, dv, q_tiles, kv_tiles, ctas;
  int first_tail_unit;     // row tiles before it were taken whole
  long long iters_base;    // the tail's flat (row tile, key tile) sequence, cut as in the main kernel
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
// give each at least two key tiles.
int choose_ctas(long long units, long long kv_tiles, int sms) {
  if (units >= sms) return sms;
  long long g = units * kv_tiles / 2;
  if (g < 1) g = 1;
  if (g > sms) g = sms;
  return static_cast<int>(g);
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
  const int ctas = choose_ctas(units, kv_tiles, device_sms());
  if (ctas_out) *ctas_out = ctas;
  // Two pieces per CTA (the ends of its range), 128 rows each, O plus (m, l).
  return static_cast<size_t>(2) * ctas * kBQ * (dv + 2);
}

int attention_tcgen05(const float* q, const void* k, const void* vt, float* o, size_t batch,
                      size_t nq, size_t nk, size_t d, size_t dv, size_t d_pitch, size_t nk_pitch,
                      AttentionArm arm, const float* v_scale, const float* k_tile_scale,
                      const float* logit_scale, bool logit_divide, bool follows_prepare,
                      float* partials, cudaStream_t s) {
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
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaSuccess;
    const void* variants[] = {reinterpret_cast<const void*>(&attention_tf32_kernel<false, Arm::TF32>),
                              reinterpret_cast<const void*>(&attention_tf32_kernel<true, Arm::TF32>),
                              reinterpret_cast<const void*>(&attention_tf32_kernel<false, Arm::BF16>),
                              reinterpret_cast<const void*>(&attention_tf32_kernel<true, Arm::BF16>),
                              reinterpret_cast<const void*>(&attention_tf32_kernel<false, Arm::MIXED>),
                              reinterpret_cast<const void*>(&attention_tf32_kernel<true, Arm::MIXED>),
                              reinterpret_cast<const void*>(&attention_tf32_kernel<false, Arm::F16>),
                              reinterpret_cast<const void*>(&attention_tf32_kernel<true, Arm::F16>)};
    for (const void* fn : variants)
      if (err == cudaSuccess)
        err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (err != cudaSuccess)
      return fail(std::string("ib_attention: cannot reserve shared memory: ") +
                  cudaGetErrorString(err));
    configured = true;
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
  int ctas = 1;
  attention_tcgen05_partial_floats(batch, nq, nk, dv, &ctas);
  if (!partials) return fail("ib_attention: workspace for partial results is missing");
  const long long units = static_cast<long long>(p.q_tiles) * p.batch;
  p.ctas = ctas;
  p.full_waves = static_cast<int>(units / ctas);
  const long long tail_units = units - static_cast<long long>(p.full_waves) * ctas;
  const long long tail_iters = tail_units * p.kv_tiles;
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
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = s;
  cfg.attrs = &overlap;
  cfg.numAttrs = g_dependent_launch && follows_prepare ? 1 : 0;
  cudaError_t launched;
  const bool prof = p.prof != nullptr;
  if (f16)
    launched = prof ? cudaLaunchKernelEx(&cfg, attention_tf32_kernel<true, Arm::F16>, map_k, map_vt, p)
                    : cudaLaunchKernelEx(&cfg, attention_tf32_kernel<false, Arm::F16>, map_k, map_vt, p);
  else if (bf16)
    launched = prof ? cudaLaunchKernelEx(&cfg, attention_tf32_kernel<true, Arm::BF16>, map_k, map_vt, p)
                    : cudaLaunchKernelEx(&cfg, attention_tf32_kernel<false, Arm::BF16>, map_k, map_vt, p);
  else if (mixed)
    launched = prof ? cudaLaunchKernelEx(&cfg, attention_tf32_kernel<true, Arm::MIXED>, map_k, map_vt, p)
                    : cudaLaunchKernelEx(&cfg, attention_tf32_kernel<false, Arm::MIXED>, map_k, map_vt, p);
  else
    launched = prof ? cudaLaunchKernelEx(&cfg, attention_tf32_kernel<true, Arm::TF32>, map_k, map_vt, p)
                    : cudaLaunchKernelEx(&cfg, attention_tf32_kernel<false, Arm::TF32>, map_k, map_vt, p);
  if (launched != cudaSuccess)
    return fail(std::string("ib_attention (tcgen05): launch failed: ") + cudaGetErrorString(launched));
  count_launch();
  // Tail row tiles shared by several CTA ranges exist unless the ranges fall on tile boundaries.
  if (tail_units > 0 && !(p.iters_rem == 0 && p.iters_base % p.kv_tiles == 0)) {
    CombineArgs a{p.part_o, p.part_m, p.part_l, o, p.nq, p.dv, p.q_tiles, p.kv_tiles, ctas,
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

// Undocumented hook for performance work: see g_attention_profile.
extern "C" void ib_debug_set_attention_profile(unsigned long long* device_counters) {
  ib::set_attention_profile(device_counters);
}
