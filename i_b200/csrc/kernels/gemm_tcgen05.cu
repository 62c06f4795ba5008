// Tensor-core contraction C[b][i][j] = sum_k A[b][i][k] * B[b][j][k]
// (`ik*jk~ijk >> +ijk~ij`, reference README.md:16; the reference's scalar nest
// is ilang-python/annotated-flashattn.c:57-89).
//
// Persistent, warp-specialised sm_100a kernel:
//   warp 0   TMA producer: 128-byte-swizzled boxes of A (128 x 32 fp32) and
//            B (BN x 32 fp32) into a 4-deep shared-memory ring
//   warp 1   MMA issuer: tcgen05.mma kind::tf32, 128 x BN x 8 per instruction,
//            fp32 accumulators in tensor memory, double-buffered per tile
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator and store it,
//            overlapping the next tile's main loop
// fp32 operands are read by the tensor core as TF32 (10-bit mantissa), products
// accumulate in fp32.  Out-of-range rows/columns/K are zero-filled by TMA and
// masked at the store, so M, N need no padding; K must be a multiple of 4
// (16-byte row pitch).  Tiles are walked in column groups so that a wave of 148
// CTAs shares its A and B panels through L2.  Outputs of at least 256 x 256 whose geometry nobody
// fixed run gemm_pair_kernel instead (further down): the same roles in each CTA of a pair that
// issues M = 256 MMAs (cta_group::2), bit-identical results.
// Roofline: tensor-bound, 2*M*N*K FLOP per batch entry.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace ib {
namespace {

using namespace sm100;

constexpr int kBM = 128;
constexpr int kBK = 32;            // fp32 per 128-byte swizzled row
constexpr int kStages = 4;
constexpr int kGroupN = 12;        // n-tiles per raster group unless the caller's geometry says otherwise
constexpr int kThreads = 192;

template <int BN>
struct Smem {
  static constexpr int kABytes = kBM * kBK * 4;
  static constexpr int kBBytes = BN * kBK * 4;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;  // + alignment slack
};

struct TileCoord {
  int batch, m_tile, n_tile;
};

// Tiles are walked in groups of `group_n` column tiles: all row tiles of a group (row tile
// outer, the group's column tiles inner) before the next group.  group_n = 1 walks column by
// column, group_n >= tiles_n row by row.
__device__ __forceinline__ TileCoord tile_coord(long long id, int tiles_m, int tiles_n, int group_n) {
  const long long per_batch = static_cast<long long>(tiles_m) * tiles_n;
  TileCoord t;
  t.batch = static_cast<int>(id / per_batch);
  long long within = id - t.batch * per_batch;
  const long long group_span = static_cast<long long>(tiles_m) * group_n;
  int group = static_cast<int>(within / group_span);
  long long in_group = within - group * group_span;
  int width = tiles_n - group * group_n;
  if (width > group_n) width = group_n;
  t.m_tile = static_cast<int>(in_group / width);
  t.n_tile = group * group_n + static_cast<int>(in_group % width);
  return t;
}

// The pointwise operators of a GemmEpilogue over the 32 consecutive columns of one row a thread
// holds.  `grow` is the row over all batch entries.  Every operator sits behind a warp-uniform
// switch inside a loop that is not unrolled, so its operands are materialised values: nothing is
// contracted into a multiply-add across operators, and the result has the bits the separate
// pointwise kernels give.
__device__ __forceinline__ void apply_epilogue(const GemmEpilogue& e, uint32_t (&r)[32], size_t grow,
                                               int col0, int n, bool vec_ok) {
#pragma unroll 1
  for (int k = 0; k < e.n_ops; ++k) {
    float t[32];
    const int w = e.which[k];
    if (w >= 0) {
      const float* p = e.operand[w];
      const int mode = e.mode[w];
      if (mode == 1 || mode == 3) {
        const float s = __ldg(mode == 1 ? p + grow : p);
#pragma unroll
        for (int v = 0; v < 32; ++v) t[v] = s;
      } else {
        const float* src = mode == 0 ? p + grow * static_cast<size_t>(n) + col0 : p + col0;
        if (vec_ok && col0 + 32 <= n && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const float4 x = __ldg(reinterpret_cast<const float4*>(src) + v);
            t[4 * v + 0] = x.x;
            t[4 * v + 1] = x.y;
            t[4 * v + 2] = x.z;
            t[4 * v + 3] = x.w;
          }
        } else {
#pragma unroll
          for (int v = 0; v < 32; ++v) t[v] = col0 + v < n ? __ldg(src + v) : 0.0f;
        }
      }
    }
    const bool right = e.acc_right[k] != 0;
#define IB_EPILOGUE_CASE(OP)                                                                   \
  case OP:                                                                                     \
    if (w < 0) {                                                                               \
      _Pragma("unroll") for (int v = 0; v < 32; ++v)                                           \
          r[v] = __float_as_uint(apply_unary(OP, __uint_as_float(r[v])));                      \
    } else if (right) {                                                                        \
      _Pragma("unroll") for (int v = 0; v < 32; ++v)                                           \
          r[v] = __float_as_uint(apply_binary(OP, t[v], __uint_as_float(r[v])));               \
    } else {                                                                                   \
      _Pragma("unroll") for (int v = 0; v < 32; ++v)                                           \
          r[v] = __float_as_uint(apply_binary(OP, __uint_as_float(r[v]), t[v]));               \
    }                                                                                          \
    break;
    switch (e.op[k]) {
      IB_EPILOGUE_CASE(IB_OP_ADD)
      IB_EPILOGUE_CASE(IB_OP_SUB)
      IB_EPILOGUE_CASE(IB_OP_MUL)
      IB_EPILOGUE_CASE(IB_OP_MAX)
      IB_EPILOGUE_CASE(IB_OP_MIN)
    }
#undef IB_EPILOGUE_CASE
  }
}

// What an epilogue thread does with 32 consecutive columns of its row: the scales of the fp16
// arm (C[i][j] = acc * row_scale[i] * col_scale[j], exact: powers of two), the caller's pointwise
// operators, the store.
__device__ __forceinline__ void finish_columns(uint32_t (&r)[32], float* crow, size_t grow, bool row_ok,
                                               float rs, const float* cs, int col0, int n, bool vec_ok,
                                               const GemmEpilogue& e) {
  if (!row_ok) return;
  if (cs) {
    if (vec_ok && col0 + 32 <= n && (reinterpret_cast<uintptr_t>(cs) & 15u) == 0) {
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const float4 w = __ldg(reinterpret_cast<const float4*>(cs + col0) + v);
        r[4 * v + 0] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r[4 * v + 0]), rs), w.x));
        r[4 * v + 1] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r[4 * v + 1]), rs), w.y));
        r[4 * v + 2] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r[4 * v + 2]), rs), w.z));
        r[4 * v + 3] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r[4 * v + 3]), rs), w.w));
      }
    } else {
#pragma unroll
      for (int v = 0; v < 32; ++v)
        if (col0 + v < n)
          r[v] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r[v]), rs), __ldg(cs + col0 + v)));
    }
  }
  if (e.n_ops) apply_epilogue(e, r, grow, col0, n, vec_ok);
  if (vec_ok && col0 + 32 <= n) {
#pragma unroll
    for (int v = 0; v < 8; ++v)
      *reinterpret_cast<float4*>(crow + col0 + 4 * v) =
          make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                      __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
  } else {
#pragma unroll
    for (int v = 0; v < 32; ++v)
      if (col0 + v < n) crow[col0 + v] = __uint_as_float(r[v]);
  }
}

// KIND selects the operand type: TF32 reads fp32 operands (32 per 128-byte row,
// K = 8 per MMA), BF16 reads bf16 operands (64 per row, K = 16 per MMA).  Either
// way one MMA consumes 32 bytes of every operand row and a stage holds 128 bytes.
template <int BN, Kind KIND>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 float* __restrict__ c, int m, int n, int k, int batch, int* status,
                 const float* __restrict__ row_scale, const float* __restrict__ col_scale,
                 int f16_operands, int group_n, const __grid_constant__ GemmEpilogue epilogue) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  using L = Smem<BN>;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * L::kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* acc_full = empty + kStages;      // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  AbortState* abort = reinterpret_cast<AbortState*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (m + kBM - 1) / kBM;
  const int tiles_n = (n + BN - 1) / BN;
  const long long total_tiles = static_cast<long long>(tiles_m) * tiles_n * batch;
  constexpr int kBKElems = KIND == Kind::TF32 ? kBK : 2 * kBK;   // elements per 128-byte row
  const int k_blocks = (k + kBKElems - 1) / kBKElems;
  constexpr uint32_t kTmemCols = 2 * BN;  // 256 or 512

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
    }
    abort->flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_descriptor(&map_a);
      tma_prefetch_descriptor(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long id = blockIdx.x; ok && id < total_tiles; id += gridDim.x) {
        const TileCoord t = tile_coord(id, tiles_m, tiles_n, group_n);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(&empty[stage], phase ^ 1, abort, status, 101))) break;
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_arrive_expect_tx(&full[stage], L::kStageBytes);
          tma_load_3d(sa, &map_a, &full[stage], kb * kBKElems, t.m_tile * kBM, t.batch);
          tma_load_3d(sb, &map_b, &full[stage], kb * kBKElems, t.n_tile * BN, t.batch);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // The 16-bit instantiation serves bf16 and fp16 operands: only the descriptor differs.
      const uint32_t idesc = KIND == Kind::BF16 && f16_operands ? make_idesc_fmt(Fmt::F16, kBM, BN)
                                                                : make_idesc(KIND, kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (long long id = blockIdx.x; ok && id < total_tiles; id += gridDim.x) {
        if (!(ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort, status, 102))) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(&full[stage], phase, abort, status, 103))) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t a_desc = make_smem_desc_sw128(sa);
          const uint64_t b_desc = make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int ks = 0; ks < kBK / 8; ++ks) {
            // 8 fp32 = 32 bytes along K inside the swizzled row: +2 in the
            // descriptor's 16-byte address units.
            mma_ss<KIND>(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc,
                               (kb | ks) != 0 ? 1u : 0u);
          }
          mma_commit(&empty[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        mma_commit(&acc_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // Epilogue warps 2..5; TMEM lane quadrant is warp % 4.
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15u) == 0);
    for (long long id = blockIdx.x; ok && id < total_tiles; id += gridDim.x) {
      const TileCoord t = tile_coord(id, tiles_m, tiles_n, group_n);
      ok = mbar_wait(&acc_full[acc], acc_phase, abort, status, 104);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = t.m_tile * kBM + quad * 32 + lane;
      float* crow = c + (static_cast<size_t>(t.batch) * m + row) * n;
      // fp16 operands stored over powers of two: C[i][j] = acc * row_scale[i] * col_scale[j], exact.
      const float rs = row_scale && row < m ? row_scale[static_cast<size_t>(t.batch) * m + row] : 1.0f;
      const float* cs = col_scale ? col_scale + static_cast<size_t>(t.batch) * n : nullptr;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);
#pragma unroll 1
      for (int chunk = 0; chunk < BN / 32; ++chunk) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + chunk * 32, r);
        tmem_wait_ld();
        const int col0 = t.n_tile * BN + chunk * 32;
        finish_columns(r, crow, static_cast<size_t>(t.batch) * m + row, row < m, rs, cs, col0, n, vec_ok,
                       epilogue);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- CTA pairs -----------------------------------------------------------------------------
// The kernel above is bound by its instruction form: an M = 128 MMA with A in shared memory
// streams A at one row per cycle, 171 cycles at N = 256 where the tensor core needs 128.  With
// cta_group::2 two CTAs of a cluster issue one M = 256 MMA: each streams its own 128 rows of A and
// holds its own 128 rows of the B tile, and the instruction takes 128 cycles (measured), the tensor
// core's rate, with operands at rest in shared memory.  Tile 256 x 256 per pair; each CTA loads a
// 128 x 32 box of A and a 128 x 32 box of B per stage (32 KB, six stages) with plain per-CTA TMA
// loads, and keeps its own 128 x 256 accumulators (two of them) in its own tensor memory.  The
// even CTA of the pair issues the MMAs.  In the running kernel an MMA takes ~160 cycles, not 128:
// per MMA a CTA's shared memory serves 12 KB of operand reads (its A, and its half of B to both
// CTAs) and takes 8 KB of TMA writes, 20 KB at 128 bytes per cycle (the single-CTA kernel moves
// 24 KB per MMA).  Measured on mm_t 8192 x 8192 x 4096: 729 against 692 TFLOP/s (TF32), 1130 against
// 1075 (scaled fp16), 1196 against 1153 (bf16); cuBLAS TF32 797 in the same run.
// What crosses between the two CTAs is barrier arrivals only:
//   peer_full[s]   a thread of the odd CTA waits for its own stage to land and arrives on the even
//                  CTA's barrier, so the issuer knows both halves of stage s are in shared memory
//                  (a relaxed arrival: with a release fence each arrival cost that thread ~1100
//                  cycles and the whole kernel ran at 304 TFLOP/s)
//   empty[s]       tcgen05.commit with cluster multicast: both CTAs' producers may refill stage s
//   acc_full[a]    the same: both CTAs' epilogue warps may read accumulator a
//   acc_empty[a]   the epilogue warps of both CTAs arrive on the even CTA's barrier (count 8)
#ifndef IB_PAIR_PROFILE
#define IB_PAIR_PROFILE 0
#endif
#if IB_PAIR_PROFILE
__device__ long long g_pair_prof[16];
#define PAIR_TICK() clock64()
#else
#define PAIR_TICK() 0ll
#endif
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = 2 * kBM * kBK * 4;      // A box + B box, 16 KB each
constexpr int kPairSmem = kPairStages * kPairStageBytes + 512 + 1024;

template <Kind KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 float* __restrict__ c, int m, int n, int k, int batch, int* status,
                 const float* __restrict__ row_scale, const float* __restrict__ col_scale,
                 int f16_operands, int group_n, const __grid_constant__ GemmEpilogue epilogue) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int BN = 256;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
  uint64_t* peer_full = full + kPairStages;
  uint64_t* empty = peer_full + kPairStages;
  uint64_t* acc_full = empty + kPairStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  AbortState* abort = reinterpret_cast<AbortState*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();   // 0 issues the MMAs
  const int pair = static_cast<int>(blockIdx.x >> 1);
  const int pairs = static_cast<int>(gridDim.x >> 1);
  const int tiles_m = (m + 2 * kBM - 1) / (2 * kBM);
  const int tiles_n = (n + BN - 1) / BN;
  const long long total_tiles = static_cast<long long>(tiles_m) * tiles_n * batch;
  constexpr int kBKElems = KIND == Kind::TF32 ? kBK : 2 * kBK;   // elements per 128-byte row
  const int k_blocks = (k + kBKElems - 1) / kBKElems;
  constexpr uint32_t kTmemCols = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&peer_full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);   // four epilogue warps in each CTA of the pair
    }
    abort->flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_alloc_permit_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();            // the peer's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_descriptor(&map_a);
      tma_prefetch_descriptor(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long w_empty = 0;
      [[maybe_unused]] const long long p_start = PAIR_TICK();
      for (long long id = pair; ok && id < total_tiles; id += pairs) {
        const TileCoord t = tile_coord(id, tiles_m, tiles_n, group_n);
        const int a_row = t.m_tile * 2 * kBM + static_cast<int>(rank) * kBM;
        const int b_row = t.n_tile * BN + static_cast<int>(rank) * kBM;
        for (int kb = 0; kb < k_blocks; ++kb) {
          const long long t0 = PAIR_TICK();
          ok = mbar_wait_cluster(&empty[stage], phase ^ 1, abort, status, 111);
          w_empty += PAIR_TICK() - t0;
          if (!ok) break;
          uint8_t* sa = smem + stage * kPairStageBytes;
          uint8_t* sb = sa + kBM * kBK * 4;
          mbar_arrive_expect_tx(&full[stage], kPairStageBytes);
          tma_load_3d(sa, &map_a, &full[stage], kb * kBKElems, a_row, t.batch);
          tma_load_3d(sb, &map_b, &full[stage], kb * kBKElems, b_row, t.batch);
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
#if IB_PAIR_PROFILE
      if (blockIdx.x < 2) {
        g_pair_prof[rank * 8 + 0] = w_empty;
        g_pair_prof[rank * 8 + 1] = PAIR_TICK() - p_start;
      }
#endif
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 1) {
      // Relay: tells the issuing CTA that this CTA's half of a stage has landed.
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long id = pair; ok && id < total_tiles; id += pairs) {
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(&full[stage], phase, abort, status, 112))) break;
          mbar_arrive_cluster_relaxed(cluster_addr_of(smem_u32(&peer_full[stage]), 0));
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    } else if (lane == 0) {
      // The 16-bit instantiation serves bf16 and fp16 operands: only the descriptor differs.
      const uint32_t idesc = KIND == Kind::BF16 && f16_operands ? make_idesc_fmt(Fmt::F16, 2 * kBM, BN)
                                                                : make_idesc(KIND, 2 * kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      long long w_full = 0, w_acc = 0, c_issue = 0;
      [[maybe_unused]] const long long i_start = PAIR_TICK();
      for (long long id = pair; ok && id < total_tiles; id += pairs) {
        long long t0 = PAIR_TICK();
        if (!(ok = mbar_wait_cluster(&acc_empty[acc], acc_phase ^ 1, abort, status, 113))) break;
        w_acc += PAIR_TICK() - t0;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          t0 = PAIR_TICK();
          if (!(ok = mbar_wait_both_cluster(&full[stage], &peer_full[stage], phase, abort, status, 114))) break;
          w_full += PAIR_TICK() - t0;
          t0 = PAIR_TICK();
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * kPairStageBytes);
          const uint64_t a_desc = make_smem_desc_sw128(sa);
          const uint64_t b_desc = make_smem_desc_sw128(sa + kBM * kBK * 4);
#pragma unroll
          for (int ks = 0; ks < kBK / 8; ++ks)
            mma_ss_pair<KIND>(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc, (kb | ks) != 0 ? 1u : 0u);
          mma_commit_pair(&empty[stage], 3);
          c_issue += PAIR_TICK() - t0;
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        mma_commit_pair(&acc_full[acc], 3);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
#if IB_PAIR_PROFILE
      if (blockIdx.x == 0) {
        g_pair_prof[2] = w_full;
        g_pair_prof[4] = w_acc;
        g_pair_prof[5] = c_issue;
        g_pair_prof[6] = PAIR_TICK() - i_start;
      }
#endif
    }
  } else {
    // Epilogue warps 2..5 of either CTA: its own 128 rows of the pair's tile.
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15u) == 0);
    for (long long id = pair; ok && id < total_tiles; id += pairs) {
      const TileCoord t = tile_coord(id, tiles_m, tiles_n, group_n);
      ok = mbar_wait_cluster(&acc_full[acc], acc_phase, abort, status, 116);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = t.m_tile * 2 * kBM + static_cast<int>(rank) * kBM + quad * 32 + lane;
      float* crow = c + (static_cast<size_t>(t.batch) * m + row) * n;
      const float rs = row_scale && row < m ? row_scale[static_cast<size_t>(t.batch) * m + row] : 1.0f;
      const float* cs = col_scale ? col_scale + static_cast<size_t>(t.batch) * n : nullptr;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);
#pragma unroll 1
      for (int chunk = 0; chunk < BN / 32; ++chunk) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + chunk * 32, r);
        tmem_wait_ld();
        const int col0 = t.n_tile * BN + chunk * 32;
        finish_columns(r, crow, static_cast<size_t>(t.batch) * m + row, row < m, rs, cs, col0, n, vec_ok,
                       epilogue);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(cluster_addr_of(smem_u32(&acc_empty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // Neither CTA may leave (or free tensor memory the pair's MMAs write) before both are done.
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <Kind KIND>
int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, float* c, size_t batch, size_t m,
                size_t n, size_t k, cudaStream_t s, int group_n, const GemmEpilogue* e,
                const float* row_scale = nullptr, const float* col_scale = nullptr,
                bool f16_operands = false) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail("ib_contract: cannot identify the current device");
  static OncePerDevice configured;
  const int rc = configured.run(dev, [] {
    cudaError_t err = cudaFuncSetAttribute(gemm_pair_kernel<KIND>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
    if (err != cudaSuccess)
      return fail(std::string("ib_contract: cannot reserve shared memory: ") + cudaGetErrorString(err));
    return 0;
  });
  if (rc == -2) return fail("ib_contract: cannot identify the current device");
  if (rc != 0) return rc;
  int* status = device_status_word(s);
  if (!status) return fail("ib_contract: cannot allocate the device status word");
  const size_t tiles = ((m + 2 * kBM - 1) / (2 * kBM)) * ((n + 255) / 256) * batch;
  int sms = kNumSMs;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t pairs = std::min(tiles, static_cast<size_t>(sms / 2));
  gemm_pair_kernel<KIND><<<static_cast<unsigned>(2 * pairs), kThreads, kPairSmem, s>>>(
      map_a, map_b, c, static_cast<int>(m), static_cast<int>(n), static_cast<int>(k),
      static_cast<int>(batch), status, row_scale, col_scale, f16_operands ? 1 : 0,
      group_n > 0 ? group_n : kGroupN, e ? *e : GemmEpilogue{});
  return check_launch("ib_contract (tcgen05 pair)");
}

template <int BN, Kind KIND>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, float* c, size_t batch, size_t m,
           size_t n, size_t k, cudaStream_t s, int group_n, const GemmEpilogue* e,
           const float* row_scale = nullptr, const float* col_scale = nullptr,
           bool f16_operands = false) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail("ib_contract: cannot identify the current device");
  // The opt-in to more than 48 KB of dynamic shared memory is per device (and per instantiation).
  static OncePerDevice configured;
  const int rc = configured.run(dev, [] {
    cudaError_t err = cudaFuncSetAttribute(gemm_tf32_kernel<BN, KIND>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           Smem<BN>::kTotal);
    if (err != cudaSuccess)
      return fail(std::string("ib_contract: cannot reserve shared memory: ") +
                  cudaGetErrorString(err));
    return 0;
  });
  if (rc == -2) return fail("ib_contract: cannot identify the current device");
  if (rc != 0) return rc;
  int* status = device_status_word(s);
  if (!status) return fail("ib_contract: cannot allocate the device status word");
  const size_t tiles = ((m + kBM - 1) / kBM) * ((n + BN - 1) / BN) * batch;
  int sms = kNumSMs;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = static_cast<int>(tiles < static_cast<size_t>(sms) ? tiles : sms);
  gemm_tf32_kernel<BN, KIND><<<grid, kThreads, Smem<BN>::kTotal, s>>>(
      map_a, map_b, c, static_cast<int>(m), static_cast<int>(n), static_cast<int>(k),
      static_cast<int>(batch), status, row_scale, col_scale, f16_operands ? 1 : 0,
      group_n > 0 ? group_n : kGroupN, e ? *e : GemmEpilogue{});
  return check_launch("ib_contract (tcgen05 tf32)");
}

}  // namespace

bool gemm_tcgen05_supported(const float* a, const float* b, const float* c, size_t m, size_t n,
                            size_t k) {
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  return aligned(a) && aligned(b) && c != nullptr && k % 4 == 0 && k >= 4 && m >= 1 && n >= 1 &&
         m < (1u << 30) && n < (1u << 30) && k < (1u << 30);
}

// Column tile: the caller's choice (128 or 256) when it gives one, else by the output's width.
static bool wide_tile(const GemmGeometry& g, size_t n) {
  return g.col_tile ? g.col_tile > 128 : n > 128;
}

// The pair kernel (256 x 256 tiles over two SMs) when nobody fixed the column tile and the output
// has room for it.  I_B200_GEMM_PAIR=0 keeps the single-CTA kernels.
static bool use_pair(const GemmGeometry& g, size_t m, size_t n) {
  static const bool enabled = [] {
    const char* v = std::getenv("I_B200_GEMM_PAIR");
    return !(v && v[0] == '0');
  }();
  return enabled && g.col_tile == 0 && m >= 256 && n >= 256;
}

int gemm_tcgen05(const float* a, const float* b, float* c, size_t batch, size_t m, size_t n,
                 size_t k, cudaStream_t s, GemmGeometry g, const GemmEpilogue* e, size_t k_parts) {
  if (batch == 0 || m == 0 || n == 0) return 0;
  if (!gemm_tcgen05_supported(a, b, c, m, n, k))
    return fail("ib_contract: shape or alignment not supported by the tensor-core arm");
  if (batch >= (1u << 30)) return fail("ib_contract: too many batch entries");
  const bool pair = use_pair(g, m, n);
  const bool wide = !pair && wide_tile(g, n);
  CUtensorMap map_a, map_b;
  size_t a_step = m * k, b_step = n * k;       // elements from one batch entry to the next
  if (k_parts > 1) {
    // The parts of the k range are the batch entries: same rows, k / k_parts columns further on.
    if (batch != 1 || k % (4 * k_parts) != 0 || e)
      return fail("ib_contract: the k range is cut for one batch entry, in multiples of four, without operators");
    batch = k_parts;
    a_step = b_step = k / k_parts;
  }
  const size_t row_pitch = k;
  if (k_parts > 1) k /= k_parts;
  if (int rc = make_tensor_map_f32(&map_a, a, batch, m, k, row_pitch, a_step, kBM)) return rc;
  if (int rc = make_tensor_map_f32(&map_b, b, batch, n, k, row_pitch, b_step, wide ? 256 : 128)) return rc;
  if (pair) return launch_pair<Kind::TF32>(map_a, map_b, c, batch, m, n, k, s, g.group_n, e);
  return wide ? launch<256, Kind::TF32>(map_a, map_b, c, batch, m, n, k, s, g.group_n, e)
              : launch<128, Kind::TF32>(map_a, map_b, c, batch, m, n, k, s, g.group_n, e);
}

int gemm_tcgen05_bf16(const void* a16, const void* b16, float* c, size_t batch, size_t m, size_t n,
                      size_t k, size_t k_pitch, cudaStream_t s, GemmGeometry g,
                      const GemmEpilogue* e) {
  if (batch == 0 || m == 0 || n == 0) return 0;
  if (k_pitch % 8 != 0 || k_pitch < k || !c || m >= (1u << 30) || n >= (1u << 30) ||
      k >= (1u << 30) || batch >= (1u << 30))
    return fail("ib_contract: shape not supported by the bf16 tensor-core arm");
  const bool pair = use_pair(g, m, n);
  const bool wide = !pair && wide_tile(g, n);
  CUtensorMap map_a, map_b;
  if (int rc = make_tensor_map_bf16(&map_a, a16, batch, m, k, k_pitch, m * k_pitch, kBM)) return rc;
  if (int rc = make_tensor_map_bf16(&map_b, b16, batch, n, k, k_pitch, n * k_pitch, wide ? 256 : 128))
    return rc;
  if (pair) return launch_pair<Kind::BF16>(map_a, map_b, c, batch, m, n, k, s, g.group_n, e);
  return wide ? launch<256, Kind::BF16>(map_a, map_b, c, batch, m, n, k, s, g.group_n, e)
              : launch<128, Kind::BF16>(map_a, map_b, c, batch, m, n, k, s, g.group_n, e);
}

int gemm_tcgen05_f16(const void* a16, const void* b16, const float* a_scale, const float* b_scale,
                     float* c, size_t batch, size_t m, size_t n, size_t k, size_t k_pitch,
                     cudaStream_t s, GemmGeometry g, const GemmEpilogue* e) {
  if (batch == 0 || m == 0 || n == 0) return 0;
  if (k_pitch % 8 != 0 || k_pitch < k || !c || !a_scale || !b_scale || m >= (1u << 30) ||
      n >= (1u << 30) || k >= (1u << 30) || batch >= (1u << 30))
    return fail("ib_contract: shape not supported by the fp16 tensor-core arm");
  const bool pair = use_pair(g, m, n);
  const bool wide = !pair && wide_tile(g, n);
  CUtensorMap map_a, map_b;
  if (int rc = make_tensor_map_bf16(&map_a, a16, batch, m, k, k_pitch, m * k_pitch, kBM)) return rc;
  if (int rc = make_tensor_map_bf16(&map_b, b16, batch, n, k, k_pitch, n * k_pitch, wide ? 256 : 128))
    return rc;
  if (pair)
    return launch_pair<Kind::BF16>(map_a, map_b, c, batch, m, n, k, s, g.group_n, e, a_scale, b_scale, true);
  return wide ? launch<256, Kind::BF16>(map_a, map_b, c, batch, m, n, k, s, g.group_n, e, a_scale, b_scale, true)
              : launch<128, Kind::BF16>(map_a, map_b, c, batch, m, n, k, s, g.group_n, e, a_scale, b_scale, true);
}

}  // namespace ib

#if IB_PAIR_PROFILE
// Development builds only (-DIB_PAIR_PROFILE=1): cycle counters of the first CTA pair.
extern "C" int ib_debug_pair_profile(long long* out16) {
  return cudaMemcpyFromSymbol(out16, ib::g_pair_prof, sizeof(long long) * 16) == cudaSuccess ? 0 : -1;
}
#endif
