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
// Q is loaded from global memory by the softmax threads, rounded to TF32 and
// stored to tensor memory once.  K/V rows past the end are zero-filled by TMA
// and masked to -inf; query rows past the end are computed and not stored.
//
// When one head has too few 128-row tiles to fill the GPU, the KV range is
// split across CTAs; each writes a normalised partial O with its (m, l) and a
// small second kernel merges them.
// Roofline: tensor-bound, 4*Nq*Nk*d FLOP per head.
#include "common.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace ib {
namespace {

using namespace sm100;

constexpr int kBQ = 128;           // query rows per CTA
constexpr int kBKV = 128;          // keys per KV tile
constexpr int kThreads = 384;
constexpr int kChunkBytes = 128 * 128;     // 128 rows x 32 fp32
constexpr int kSlotBytes = 4 * kChunkBytes;
constexpr int kRing = 3;
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
  int splits;          // KV splits per tile
  int kv_tiles;        // 128-key tiles per head
  int kv_per_split;
  float* o;            // [batch][nq][dv]
  float* part_o;       // [splits][batch][nq][dv] when splits > 1
  float* part_m;       // [splits][batch][nq]
  float* part_l;
  int* status;
  unsigned long long* prof;   // optional per-CTA wait-cycle counters (debugging aid), or null
};

struct Shared {
  uint64_t kv_full[kRing];
  uint64_t kv_empty[kRing];
  uint64_t q_ready;
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t pv_done[2];       // [KV tile parity]: see the note at its wait
  uint32_t tmem_slot;
  AbortState abort;
  int give_up;               // raised before a named barrier, read after it
  float half_max[2][2][kBQ]; // [iteration parity][warpgroup][row]
  float half_sum[2][kBQ];
};

__device__ __forceinline__ void softmax_pair_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
attention_tf32_kernel(const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_vt, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* ring = smem;                                     // [kRing][64 KB]
  Shared* sh = reinterpret_cast<Shared*>(ring + kRing * kSlotBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int d_chunks = (p.d + 31) / 32;

  // Work unit of this CTA.
  int unit = blockIdx.x;
  const int split = unit % p.splits;
  unit /= p.splits;
  const int qt = unit % p.q_tiles;
  const int b = unit / p.q_tiles;
  const int kv_lo = split * p.kv_per_split;
  const int kv_hi = min(p.kv_tiles, kv_lo + p.kv_per_split);
  const int n_kv = kv_hi - kv_lo;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&sh->kv_full[s], 1);
      mbar_init(&sh->kv_empty[s], 1);
    }
    mbar_init(&sh->q_ready, 8);            // one arrival per softmax warp
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

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      tma_prefetch_descriptor(&map_k);
      tma_prefetch_descriptor(&map_vt);
      int slot = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long waited = 0;
      auto load_k = [&](int j) {
        const long long t0 = clock64();
        if (!(ok = mbar_wait(&sh->kv_empty[slot], phase ^ 1, abort, p.status, 201))) return;
        waited += clock64() - t0;
        uint8_t* dst = ring + slot * kSlotBytes;
        mbar_arrive_expect_tx(&sh->kv_full[slot], d_chunks * kChunkBytes);
        for (int c = 0; c < d_chunks; ++c)
          tma_load_3d(dst + c * kChunkBytes, &map_k, &sh->kv_full[slot], c * 32, j * kBKV, b);
        if (++slot == kRing) { slot = 0; phase ^= 1; }
      };
      auto load_v = [&](int j) {
        const long long t0 = clock64();
        if (!(ok = mbar_wait(&sh->kv_empty[slot], phase ^ 1, abort, p.status, 202))) return;
        waited += clock64() - t0;
        uint8_t* dst = ring + slot * kSlotBytes;
        mbar_arrive_expect_tx(&sh->kv_full[slot], 4 * kChunkBytes);
        for (int c = 0; c < 4; ++c)
          tma_load_3d(dst + c * kChunkBytes, &map_vt, &sh->kv_full[slot], j * kBKV + c * 32, 0, b);
        if (++slot == kRing) { slot = 0; phase ^= 1; }
      };
      // Consumption order: K(0), then per tile K(j+1) before V(j).
      load_k(kv_lo);
      for (int jj = 0; ok && jj < n_kv; ++jj) {
        if (jj + 1 < n_kv) load_k(kv_lo + jj + 1);
        if (ok) load_v(kv_lo + jj);
      }
      if (p.prof) p.prof[blockIdx.x * 8 + 0] = waited;
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      const uint32_t idesc_qk = make_idesc(Kind::TF32, kBQ, kBKV);
      const uint32_t n_pv = static_cast<uint32_t>((p.dv + 15) / 16 * 16);
      const uint32_t idesc_pv = make_idesc(Kind::TF32, kBQ, n_pv);
      const int k_steps = (p.d + 7) / 8;
      int slot = 0;
      uint32_t phase = 0;
      const uint32_t ring_addr = smem_u32(ring);
      long long wait_k = 0, wait_v = 0, wait_p = 0, issue_qk_cycles = 0, issue_pv_cycles = 0;
      const long long t_start = clock64();
      bool ok = mbar_wait(&sh->q_ready, 0, abort, p.status, 203);
      tc_fence_after_sync();

      // S[buf] = Q K^T from the K tile in the current slot (A = Q in tensor memory).
      auto issue_qk = [&](int buf) {
        const long long t0 = clock64();
        if (!(ok = mbar_wait(&sh->kv_full[slot], phase, abort, p.status, 204))) return;
        wait_k += clock64() - t0;
        tc_fence_after_sync();
        // One descriptor per slot; a K step moves it by a compile-time constant
        // (32 bytes inside the swizzled row, 16 KB to the next 32-feature chunk),
        // so the issuing thread spends one 64-bit add per MMA.
        const long long ti = clock64();
        const uint64_t k_desc = make_smem_desc_sw128(ring_addr + slot * kSlotBytes);
        const uint32_t d_tmem = tmem_base + kTmemS + static_cast<uint32_t>(buf * kBKV);
        const uint32_t q_tmem = tmem_base + kTmemQ;
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {
          if (ks < k_steps)
            mma_ts<Kind::TF32>(d_tmem, q_tmem + ks * 8,
                               k_desc + (((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4), idesc_qk,
                               ks != 0 ? 1u : 0u);
        }
        mma_commit(&sh->s_full[buf]);
        mma_commit(&sh->kv_empty[slot]);
        issue_qk_cycles += clock64() - ti;
        if (++slot == kRing) { slot = 0; phase ^= 1; }
      };
      // O += P[buf] V from the V^T tile in the current slot (A = P in tensor memory).
      auto issue_pv = [&](int jj) {
        const int buf = jj & 1;
        long long t0 = clock64();
        if (!(ok = mbar_wait(&sh->kv_full[slot], phase, abort, p.status, 205))) return;
        wait_v += clock64() - t0;
        t0 = clock64();
        if (!(ok = mbar_wait(&sh->p_full[buf], (jj >> 1) & 1, abort, p.status, 206))) return;
        wait_p += clock64() - t0;
        tc_fence_after_sync();
        const long long ti = clock64();
        const uint64_t v_desc = make_smem_desc_sw128(ring_addr + slot * kSlotBytes);
        const uint32_t d_tmem = tmem_base + kTmemO;
        const uint32_t p_tmem = tmem_base + kTmemS + static_cast<uint32_t>(buf * kBKV);
        if (jj == 0) {
          mma_ts<Kind::TF32>(d_tmem, p_tmem, v_desc, idesc_pv, 0u);
        } else {
          mma_ts<Kind::TF32>(d_tmem, p_tmem, v_desc, idesc_pv, 1u);
        }
#pragma unroll
        for (int ks = 1; ks < kBKV / 8; ++ks)
          mma_ts<Kind::TF32>(d_tmem, p_tmem + ks * 8,
                             v_desc + (((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4), idesc_pv, 1u);
        mma_commit(&sh->pv_done[buf]);
        mma_commit(&sh->kv_empty[slot]);
        issue_pv_cycles += clock64() - ti;
        if (++slot == kRing) { slot = 0; phase ^= 1; }
      };

      if (ok) issue_qk(0);
      for (int jj = 0; ok && jj < n_kv; ++jj) {
        if (jj + 1 < n_kv) issue_qk((jj + 1) & 1);
        if (ok) issue_pv(jj);
      }
      if (p.prof) {
        p.prof[blockIdx.x * 8 + 1] = wait_k;
        p.prof[blockIdx.x * 8 + 2] = wait_v;
        p.prof[blockIdx.x * 8 + 5] = issue_qk_cycles;
        p.prof[blockIdx.x * 8 + 6] = issue_pv_cycles;
        p.prof[blockIdx.x * 8 + 3] = wait_p;
        p.prof[blockIdx.x * 8 + 4] = clock64() - t_start;
      }
    }
  } else if (warp >= 4 && n_kv > 0) {
    const int h = (warp - 4) >> 2;            // column half of this warpgroup
    const int quad = warp & 3;                // TMEM lane quadrant
    const int r = quad * 32 + lane;           // row within the tile
    const long long row = static_cast<long long>(qt) * kBQ + r;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t o_tmem = tmem_base + lane_bits + kTmemO;
    const int dv_chunks = (p.dv + 31) / 32;

    // ---- Q: global -> TF32 (nearest) -> tensor memory, columns [64h, 64h+64) ----
    {
      const float* qrow = p.q + (static_cast<size_t>(b) * p.nq + row) * p.d;
      const bool live = row < p.nq;
      const bool vec = (reinterpret_cast<uintptr_t>(p.q) & 15u) == 0 && p.d % 4 == 0;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col0 = h * 64 + c * 32;
        uint32_t v[32];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          if (live && vec && col0 + e + 4 <= p.d) {
            x = *reinterpret_cast<const float4*>(qrow + col0 + e);
          } else if (live) {
            if (col0 + e + 0 < p.d) x.x = qrow[col0 + e + 0];
            if (col0 + e + 1 < p.d) x.y = qrow[col0 + e + 1];
            if (col0 + e + 2 < p.d) x.z = qrow[col0 + e + 2];
            if (col0 + e + 3 < p.d) x.w = qrow[col0 + e + 3];
          }
          asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v[e + 0]) : "f"(x.x));
          asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v[e + 1]) : "f"(x.y));
          asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v[e + 2]) : "f"(x.z));
          asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v[e + 3]) : "f"(x.w));
        }
        tmem_st_32x32(tmem_base + lane_bits + kTmemQ + col0, v);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->q_ready);
    }

    float m_used = -CUDART_INF_F;             // running maximum, log2 domain
    float l = 0.0f;                           // this half's share of the row sum
    bool dead = false;                        // a wait gave up; keep hitting the barriers only
    long long wait_s = 0;
    const long long t_start = clock64();

    for (int jj = 0; jj < n_kv; ++jj) {
      const int buf = jj & 1;
      const uint32_t s_tmem = tmem_base + lane_bits + kTmemS + static_cast<uint32_t>(buf * kBKV) +
                              static_cast<uint32_t>(h * 64);
      uint32_t s0[32], s1[32];
      if (!dead) {
        const long long t0 = clock64();
        dead = !mbar_wait_warp(&sh->s_full[buf], (jj >> 1) & 1, abort, p.status, 207);
        wait_s += clock64() - t0;
      }
      float mx = -CUDART_INF_F;
      if (!dead) {
        tc_fence_after_sync();
        tmem_ld_32x32(s_tmem, s0);
        tmem_ld_32x32(s_tmem + 32, s1);
        tmem_wait_ld();
        const int col0 = (kv_lo + jj) * kBKV + h * 64;
        if (col0 + 64 > p.nk) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (col0 + c >= p.nk) s0[c] = __float_as_uint(-CUDART_INF_F);
            if (col0 + 32 + c >= p.nk) s1[c] = __float_as_uint(-CUDART_INF_F);
          }
        }
        float mx0 = -CUDART_INF_F, mx1 = mx0, mx2 = mx0, mx3 = mx0;
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          mx0 = fmaxf(mx0, __uint_as_float(s0[c]));
          mx1 = fmaxf(mx1, __uint_as_float(s0[c + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(s1[c]));
          mx3 = fmaxf(mx3, __uint_as_float(s1[c + 1]));
        }
        mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        sh->half_max[buf][h][r] = mx;
      } else {
        sh->give_up = 1;
      }
      softmax_pair_sync();
      if (sh->give_up) break;                 // uniform: every writer wrote before the barrier
      mx = fmaxf(mx, sh->half_max[buf][h ^ 1][r]);

      const float m_new = fmaxf(m_used, mx * kLog2E32);
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
          dead = !mbar_wait_warp(&sh->pv_done[(jj - 1) & 1], ((jj - 1) >> 1) & 1, abort, p.status,
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
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float e0 = ex2_approx(fmaf(__uint_as_float(s0[c]), kLog2E32, -m_used));
        float e1 = ex2_approx(fmaf(__uint_as_float(s1[c]), kLog2E32, -m_used));
        sum0 += e0;
        sum1 += e1;
        s0[c] = __float_as_uint(e0);
        s1[c] = __float_as_uint(e1);
      }
      l += sum0 + sum1;
      tmem_st_32x32(s_tmem, s0);
      tmem_st_32x32(s_tmem + 32, s1);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->p_full[buf]);
    }

    if (p.prof && quad == 0 && lane == 0) {
      if (h == 0) p.prof[blockIdx.x * 8 + 7] = clock64() - t_start - wait_s;
    }

    // ---- epilogue: total row sum, normalise, store columns [64h, 64h+64) of O ----
    if (!sh->give_up && !dead) {
      dead = !mbar_wait_warp(&sh->pv_done[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort, p.status,
                             209);
    }
    sh->half_sum[h][r] = l;
    if (dead) sh->give_up = 1;
    softmax_pair_sync();
    if (!sh->give_up) {
      tc_fence_after_sync();
      const float l_total = l + sh->half_sum[h ^ 1][r];
      const float inv = 1.0f / l_total;
      float* dst;
      if (p.splits == 1) {
        dst = p.o + (static_cast<size_t>(b) * p.nq + row) * p.dv;
      } else {
        const size_t prow = (static_cast<size_t>(split) * p.batch + b) * p.nq + row;
        dst = p.part_o + prow * p.dv;
        if (row < p.nq && h == 0) {
          p.part_m[prow] = m_used;
          p.part_l[prow] = l_total;
        }
      }
      const bool vec_ok = (p.dv % 4 == 0) && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
      for (int c = h * 2; c < h * 2 + 2 && c < dv_chunks; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(o_tmem + c * 32, o);
        tmem_wait_ld();
        if (row < p.nq) {
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
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Merges KV-split partials: O = sum_s w_s O_s / sum_s w_s, w_s = l_s 2^(m_s - max m).
// One thread per four output columns; dv4 = ceil(dv / 4).
__global__ void __launch_bounds__(256)
attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_m,
                         const float* __restrict__ part_l, float* __restrict__ o, size_t rows,
                         int dv, int splits, bool vec) {
  const int dv4 = (dv + 3) / 4;
  const size_t total = rows * dv4;
  const size_t stride = static_cast<size_t>(gridDim.x) * 256;
  for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += stride) {
    const size_t r = i / dv4;
    const int c = static_cast<int>(i - r * dv4) * 4;
    float m = -CUDART_INF_F;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, part_m[s * rows + r]);
    float wsum = 0.0f;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int s = 0; s < splits; ++s) {
      const float w = part_l[s * rows + r] * exp2f(part_m[s * rows + r] - m);
      wsum += w;
      const float* src = part_o + (s * rows + r) * dv + c;
      if (vec) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(src));
        acc[0] += w * v.x; acc[1] += w * v.y; acc[2] += w * v.z; acc[3] += w * v.w;
      } else {
        for (int e = 0; e < 4 && c + e < dv; ++e) acc[e] += w * src[e];
      }
    }
    const float inv = 1.0f / wsum;
    float* dst = o + r * dv + c;
    if (vec) {
      *reinterpret_cast<float4*>(dst) = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
    } else {
      for (int e = 0; e < 4 && c + e < dv; ++e) dst[e] = acc[e] * inv;
    }
  }
}

// Debugging aid: when set (device pointer to 8 counters per CTA), the kernel
// records how many cycles each role spent waiting on its barriers.
unsigned long long* g_attention_profile = nullptr;

int choose_splits(size_t units, int kv_tiles, int sms) {
  if (units >= static_cast<size_t>(sms) || kv_tiles < 8) return 1;
  int s = static_cast<int>(sms / units);
  if (s < 1) s = 1;
  if (s > kv_tiles / 4) s = kv_tiles / 4;
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

}  // namespace

void set_attention_profile(unsigned long long* p) { g_attention_profile = p; }

size_t attention_tcgen05_partial_floats(size_t batch, size_t nq, size_t nk, size_t dv, int* splits_out) {
  int sms = kNumSMs;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t q_tiles = (nq + kBQ - 1) / kBQ;
  const int kv_tiles = static_cast<int>((nk + kBKV - 1) / kBKV);
  const int splits = choose_splits(q_tiles * batch, kv_tiles, sms);
  if (splits_out) *splits_out = splits;
  if (splits == 1) return 0;
  return static_cast<size_t>(splits) * batch * nq * (dv + 2);
}

int attention_tcgen05(const float* q, const float* k, const float* vt, float* o, size_t batch,
                      size_t nq, size_t nk, size_t d, size_t dv, size_t nk_pitch, float* partials,
                      cudaStream_t s) {
  if (batch == 0 || nq == 0) return 0;
  if (nk == 0) return fail("ib_attention: no keys");
  if (nq >= (1u << 30) || nk >= (1u << 30) || batch >= (1u << 20))
    return fail("ib_attention: shape too large");
  if (d % 4 != 0 || d < 4 || d > 128 || dv < 1 || dv > 128)
    return fail("ib_attention: head dimensions outside the fused kernel's range");
  const int smem_bytes = 1024 + kRing * kSlotBytes + static_cast<int>(sizeof(Shared)) + 64;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_tf32_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
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
  int splits = 1;
  attention_tcgen05_partial_floats(batch, nq, nk, dv, &splits);
  if (splits > 1 && !partials) return fail("ib_attention: workspace for KV splits is missing");
  p.splits = splits;
  p.kv_per_split = (p.kv_tiles + splits - 1) / splits;
  // Every split must own at least one KV tile.
  while (p.splits > 1 && (p.splits - 1) * p.kv_per_split >= p.kv_tiles) --p.splits;
  p.o = o;
  if (p.splits > 1) {
    const size_t rows = static_cast<size_t>(p.splits) * batch * nq;
    p.part_o = partials;
    p.part_m = partials + rows * dv;
    p.part_l = p.part_m + rows;
  }
  p.status = device_status_word(s);
  if (!p.status) return fail("ib_attention: cannot allocate the device status word");
  p.prof = g_attention_profile;

  CUtensorMap map_k, map_vt;
  if (int rc = make_tensor_map_f32(&map_k, k, batch, nk, d, d, nk * d, kBKV)) return rc;
  if (int rc = make_tensor_map_f32(&map_vt, vt, batch, dv, nk, nk_pitch, dv * nk_pitch, 128))
    return rc;

  const size_t grid = static_cast<size_t>(p.q_tiles) * p.splits * batch;
  if (grid >= (1u << 31)) return fail("ib_attention: too many work units");
  attention_tf32_kernel<<<static_cast<unsigned>(grid), kThreads, smem_bytes, s>>>(map_k, map_vt, p);
  if (int rc = check_launch("ib_attention (tcgen05 tf32)")) return rc;
  if (p.splits > 1) {
    const size_t rows = batch * nq;
    size_t blocks = (rows * ((dv + 3) / 4) + 255) / 256;
    if (blocks > static_cast<size_t>(kNumSMs) * 16) blocks = static_cast<size_t>(kNumSMs) * 16;
    const bool vec = dv % 4 == 0 && (reinterpret_cast<uintptr_t>(o) & 15u) == 0 &&
                     (reinterpret_cast<uintptr_t>(p.part_o) & 15u) == 0;
    attention_combine_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        p.part_o, p.part_m, p.part_l, o, rows, p.dv, p.splits, vec);
    return check_launch("ib_attention (combine)");
  }
  return 0;
}

}  // namespace ib

// Undocumented hook for performance work: see g_attention_profile.
extern "C" void ib_debug_set_attention_profile(unsigned long long* device_counters) {
  ib::set_attention_profile(device_counters);
}
