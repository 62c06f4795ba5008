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
// Layout of one CTA (384 threads, 256 query rows = two 128-row tiles):
//   warp 0      TMA producer.  Q tiles once; then K and V^T tiles of 64 keys
//               through a ring of 32 KB slots (128-byte swizzled rows).
//   warp 1      MMA issuer.  S[t] = Q[t] K^T with tcgen05.mma kind::tf32
//               (A, B from shared memory), O[t] += P[t] V with A = P read from
//               tensor memory.  S is double-buffered per tile so the QK^T of
//               the next KV tile runs while the softmax of this one is in
//               flight.
//   warps 4-7   softmax for tile 0, warps 8-11 for tile 1: one thread per
//               query row; S is read from tensor memory, P written back over
//               it; the row maximum/sum live in registers.  O is rescaled in
//               tensor memory only when the maximum grows by more than 2^8.
// Tensor memory: S[tile][buf] 4 x 64 columns, O[tile] 2 x 128 columns.
// K/V rows past the end are zero-filled by TMA and masked to -inf; query rows
// past the end are computed and not stored.
//
// When one head has too few 256-row blocks to fill the GPU, the KV range is
// split across CTAs; each writes a normalised partial O with its (m, l) and a
// small second kernel merges them.
// Roofline: tensor-bound, 4*Nq*Nk*d FLOP per head.
#include "common.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace ib {
namespace {

using namespace sm100;

constexpr int kBQ = 128;          // rows per query tile
constexpr int kBKV = 64;          // keys per KV tile
constexpr int kThreads = 384;
constexpr int kQChunkBytes = kBQ * 128;    // 128 rows x 32 fp32
constexpr int kKChunkBytes = kBKV * 128;   // 64 rows x 32 fp32
constexpr int kVChunkBytes = 128 * 128;    // 128 dv rows x 32 keys
constexpr int kSlotBytes = 32768;
constexpr int kMaxRing = 8;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemS = 0;             // + (tile * 2 + buf) * 64
constexpr uint32_t kTmemO = 256;           // + tile * 128
constexpr float kLog2E32 = 1.4426950216293335f;  // log2(2.71828175f)
constexpr float kRescaleThreshold = 8.0f;

struct Params {
  int nq, nk, d, dv, batch;
  int q_blocks;        // 256-row blocks per head
  int splits;          // KV splits per block
  int kv_blocks;       // 64-key tiles per head
  int kv_per_split;
  int ring;            // ring slots
  float* o;            // [batch][nq][dv]
  float* part_o;       // [splits][batch][nq][dv] when splits > 1
  float* part_m;       // [splits][batch][nq]
  float* part_l;
  int* status;
  unsigned long long* prof;   // optional per-CTA wait-cycle counters (debugging aid), or null
};

struct Barriers {
  uint64_t q_full;
  uint64_t kv_full[kMaxRing];
  uint64_t kv_empty[kMaxRing];
  uint64_t s_full[2][2];
  uint64_t p_full[2][2];
  uint64_t pv_done[2][2];   // [tile][KV tile parity]: see the note at its wait
  uint32_t tmem_slot;
  AbortState abort;
};

__global__ void __launch_bounds__(kThreads, 1)
attention_tf32_kernel(const __grid_constant__ CUtensorMap map_q,
                      const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_vt, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int d_chunks = (p.d + 31) / 32;
  uint8_t* q_smem = smem;                                   // [2][d_chunks][128 rows][128 B]
  uint8_t* ring = q_smem + 2 * d_chunks * kQChunkBytes;     // [ring][32 KB]
  Barriers* bars = reinterpret_cast<Barriers*>(ring + p.ring * kSlotBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Work unit of this CTA.
  int unit = blockIdx.x;
  const int split = unit % p.splits;
  unit /= p.splits;
  const int qb = unit % p.q_blocks;
  const int b = unit / p.q_blocks;
  const int kv_lo = split * p.kv_per_split;
  const int kv_hi = min(p.kv_blocks, kv_lo + p.kv_per_split);
  const int n_kv = kv_hi - kv_lo;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < p.ring; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      for (int u = 0; u < 2; ++u) {
        mbar_init(&bars->s_full[t][u], 1);
        mbar_init(&bars->p_full[t][u], 4);   // one arrival per softmax warp
        mbar_init(&bars->pv_done[t][u], 1);
      }
    }
    bars->abort.flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_slot, kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_slot;
  AbortState* abort = &bars->abort;

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      tma_prefetch_descriptor(&map_q);
      tma_prefetch_descriptor(&map_k);
      tma_prefetch_descriptor(&map_vt);
      mbar_arrive_expect_tx(&bars->q_full, 2 * d_chunks * kQChunkBytes);
      for (int t = 0; t < 2; ++t)
        for (int c = 0; c < d_chunks; ++c)
          tma_load_3d(q_smem + (t * d_chunks + c) * kQChunkBytes, &map_q, &bars->q_full, c * 32,
                      qb * 2 * kBQ + t * kBQ, b);
      int slot = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long waited = 0;
      auto load_k = [&](int j) {
        const long long t0 = clock64();
        if (!(ok = mbar_wait(&bars->kv_empty[slot], phase ^ 1, abort, p.status, 201))) return;
        waited += clock64() - t0;
        uint8_t* dst = ring + slot * kSlotBytes;
        mbar_arrive_expect_tx(&bars->kv_full[slot], d_chunks * kKChunkBytes);
        for (int c = 0; c < d_chunks; ++c)
          tma_load_3d(dst + c * kKChunkBytes, &map_k, &bars->kv_full[slot], c * 32, j * kBKV, b);
        if (++slot == p.ring) { slot = 0; phase ^= 1; }
      };
      auto load_v = [&](int j) {
        const long long t0 = clock64();
        if (!(ok = mbar_wait(&bars->kv_empty[slot], phase ^ 1, abort, p.status, 202))) return;
        waited += clock64() - t0;
        uint8_t* dst = ring + slot * kSlotBytes;
        mbar_arrive_expect_tx(&bars->kv_full[slot], 2 * kVChunkBytes);
        for (int c = 0; c < 2; ++c)
          tma_load_3d(dst + c * kVChunkBytes, &map_vt, &bars->kv_full[slot], j * kBKV + c * 32, 0,
                      b);
        if (++slot == p.ring) { slot = 0; phase ^= 1; }
      };
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
      bool ok = mbar_wait(&bars->q_full, 0, abort, p.status, 203);
      const uint32_t q_addr = smem_u32(q_smem);
      const uint32_t ring_addr = smem_u32(ring);

      // S[t][buf] = Q[t] K^T for both tiles from the K tile in the current slot.
      long long wait_k = 0, wait_v = 0, wait_p = 0;
      const long long t_start = clock64();
      auto issue_qk = [&](int buf) {
        const long long t0 = clock64();
        if (!(ok = mbar_wait(&bars->kv_full[slot], phase, abort, p.status, 204))) return;
        wait_k += clock64() - t0;
        tc_fence_after_sync();
        const uint32_t k_addr = ring_addr + slot * kSlotBytes;
        for (int t = 0; t < 2; ++t) {
          const uint32_t d_tmem = tmem_base + kTmemS + static_cast<uint32_t>((t * 2 + buf) * kBKV);
          for (int ks = 0; ks < k_steps; ++ks) {
            const int c = ks >> 2, r = ks & 3;
            const uint64_t a_desc =
                make_smem_desc_sw128(q_addr + (t * d_chunks + c) * kQChunkBytes + r * 32);
            const uint64_t b_desc = make_smem_desc_sw128(k_addr + c * kKChunkBytes + r * 32);
            mma_ss<Kind::TF32>(d_tmem, a_desc, b_desc, idesc_qk, ks != 0 ? 1u : 0u);
          }
          mma_commit(&bars->s_full[t][buf]);
        }
        mma_commit(&bars->kv_empty[slot]);
        if (++slot == p.ring) { slot = 0; phase ^= 1; }
      };
      // O[t] += P[t][buf] V for both tiles from the V^T tile in the current slot.
      auto issue_pv = [&](int jj) {
        const int buf = jj & 1;
        long long t0 = clock64();
        if (!(ok = mbar_wait(&bars->kv_full[slot], phase, abort, p.status, 205))) return;
        wait_v += clock64() - t0;
        const uint32_t v_addr = ring_addr + slot * kSlotBytes;
        for (int t = 0; t < 2; ++t) {
          t0 = clock64();
          if (!(ok = mbar_wait(&bars->p_full[t][buf], (jj >> 1) & 1, abort, p.status, 206))) return;
          wait_p += clock64() - t0;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + kTmemO + static_cast<uint32_t>(t * 128);
          const uint32_t p_tmem = tmem_base + kTmemS + static_cast<uint32_t>((t * 2 + buf) * kBKV);
#pragma unroll
          for (int ks = 0; ks < kBKV / 8; ++ks) {
            const int c = ks >> 2, r = ks & 3;
            const uint64_t b_desc = make_smem_desc_sw128(v_addr + c * kVChunkBytes + r * 32);
            mma_ts<Kind::TF32>(d_tmem, p_tmem + ks * 8, b_desc, idesc_pv,
                               (jj | ks) != 0 ? 1u : 0u);
          }
          mma_commit(&bars->pv_done[t][buf]);
        }
        mma_commit(&bars->kv_empty[slot]);
        if (++slot == p.ring) { slot = 0; phase ^= 1; }
      };

      if (ok) issue_qk(0);
      for (int jj = 0; ok && jj < n_kv; ++jj) {
        if (jj + 1 < n_kv) issue_qk((jj + 1) & 1);
        if (ok) issue_pv(jj);
      }
      if (p.prof) {
        p.prof[blockIdx.x * 8 + 1] = wait_k;
        p.prof[blockIdx.x * 8 + 2] = wait_v;
        p.prof[blockIdx.x * 8 + 3] = wait_p;
        p.prof[blockIdx.x * 8 + 4] = clock64() - t_start;
      }
    }
  } else if (warp >= 4 && n_kv > 0) {
    const int t = (warp - 4) >> 2;            // query tile of this warpgroup
    const int quad = warp & 3;                // TMEM lane quadrant
    const int row_in_tile = quad * 32 + lane;
    const long long row = static_cast<long long>(qb) * 2 * kBQ + t * kBQ + row_in_tile;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t o_tmem = tmem_base + lane_bits + kTmemO + static_cast<uint32_t>(t * 128);
    const int dv_chunks = (p.dv + 31) / 32;
    float m_used = -CUDART_INF_F;             // running maximum, log2 domain
    float l = 0.0f;
    bool ok = true;

    long long wait_s = 0;
    const long long t_start = clock64();
    for (int jj = 0; jj < n_kv; ++jj) {
      const int buf = jj & 1;
      const long long t0 = clock64();
      ok = mbar_wait(&bars->s_full[t][buf], (jj >> 1) & 1, abort, p.status, 207);
      wait_s += clock64() - t0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t s_tmem = tmem_base + lane_bits + kTmemS + static_cast<uint32_t>((t * 2 + buf) * kBKV);
      uint32_t s0[32], s1[32];
      tmem_ld_32x32(s_tmem, s0);
      tmem_ld_32x32(s_tmem + 32, s1);
      tmem_wait_ld();

      const int col0 = (kv_lo + jj) * kBKV;
      if (col0 + kBKV > p.nk) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          if (col0 + c >= p.nk) s0[c] = __float_as_uint(-CUDART_INF_F);
          if (col0 + 32 + c >= p.nk) s1[c] = __float_as_uint(-CUDART_INF_F);
        }
      }
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int c = 0; c < 32; ++c)
        mx = fmaxf(mx, fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])));
      const float m_new = fmaxf(m_used, mx * kLog2E32);
      const bool grow = m_new > m_used + kRescaleThreshold;
      if (__any_sync(0xffffffffu, grow)) {
        const float factor = grow ? ex2_approx(m_used - m_new) : 1.0f;
        if (grow) m_used = m_new;
        l *= factor;
        if (jj > 0) {
          // O[t] may still be receiving P V of the previous KV tile.  Its
          // completion is signalled on the barrier of that tile's parity, so a
          // waiter that skipped earlier phases is never more than one phase
          // behind (a parity wait cannot tell phases two apart).
          ok = mbar_wait(&bars->pv_done[t][(jj - 1) & 1], ((jj - 1) >> 1) & 1, abort, p.status,
                         208);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          for (int c = 0; c < dv_chunks; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(o_tmem + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
            tmem_st_32x32(o_tmem + c * 32, o);
          }
        }
      }
      float sum = 0.0f;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float e0 = ex2_approx(fmaf(__uint_as_float(s0[c]), kLog2E32, -m_used));
        float e1 = ex2_approx(fmaf(__uint_as_float(s1[c]), kLog2E32, -m_used));
        sum += e0 + e1;
        s0[c] = __float_as_uint(e0);
        s1[c] = __float_as_uint(e1);
      }
      l += sum;
      tmem_st_32x32(s_tmem, s0);
      tmem_st_32x32(s_tmem + 32, s1);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[t][buf]);
    }

    if (p.prof && (warp & 3) == 0 && lane == 0) {
      p.prof[blockIdx.x * 8 + 5 + t] = wait_s;
      if (t == 0) p.prof[blockIdx.x * 8 + 7] = clock64() - t_start;
    }
    if (ok) {
      ok = mbar_wait(&bars->pv_done[t][(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort, p.status,
                     209);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.0f / l;
      float* dst;
      if (p.splits == 1) {
        dst = p.o + (static_cast<size_t>(b) * p.nq + row) * p.dv;
      } else {
        const size_t prow = (static_cast<size_t>(split) * p.batch + b) * p.nq + row;
        dst = p.part_o + prow * p.dv;
        if (row < p.nq) {
          p.part_m[prow] = m_used;
          p.part_l[prow] = l;
        }
      }
      const bool vec_ok = (p.dv % 4 == 0) && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
      for (int c = 0; c < dv_chunks; ++c) {
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

int choose_splits(size_t units, int kv_blocks, int sms) {
  if (units >= static_cast<size_t>(sms) || kv_blocks < 8) return 1;
  int s = static_cast<int>(sms / units);
  if (s < 1) s = 1;
  if (s > kv_blocks / 4) s = kv_blocks / 4;
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

}  // namespace

void set_attention_profile(unsigned long long* p) { g_attention_profile = p; }

bool attention_tcgen05_supported(const float* q, const float* k, const float* o, size_t d,
                                 size_t dv) {
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  return aligned(q) && aligned(k) && o != nullptr && d % 4 == 0 && d >= 4 && d <= 128 && dv >= 1 &&
         dv <= 128;
}

size_t attention_tcgen05_partial_floats(size_t batch, size_t nq, size_t nk, size_t dv, int* splits_out) {
  int sms = kNumSMs;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t q_blocks = (nq + 2 * kBQ - 1) / (2 * kBQ);
  const int kv_blocks = static_cast<int>((nk + kBKV - 1) / kBKV);
  const int splits = choose_splits(q_blocks * batch, kv_blocks, sms);
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
  static bool configured = false;
  static int max_smem = 0;
  if (!configured) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaError_t err = cudaFuncSetAttribute(attention_tf32_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (err != cudaSuccess)
      return fail(std::string("ib_attention: cannot reserve shared memory: ") +
                  cudaGetErrorString(err));
    configured = true;
  }
  Params p{};
  p.nq = static_cast<int>(nq);
  p.nk = static_cast<int>(nk);
  p.d = static_cast<int>(d);
  p.dv = static_cast<int>(dv);
  p.batch = static_cast<int>(batch);
  p.q_blocks = static_cast<int>((nq + 2 * kBQ - 1) / (2 * kBQ));
  p.kv_blocks = static_cast<int>((nk + kBKV - 1) / kBKV);
  int splits = 1;
  const size_t part_floats = attention_tcgen05_partial_floats(batch, nq, nk, dv, &splits);
  if (splits > 1 && !partials) return fail("ib_attention: workspace for KV splits is missing");
  p.splits = splits;
  p.kv_per_split = (p.kv_blocks + splits - 1) / splits;
  // Every split must own at least one KV tile.
  while (p.splits > 1 && (p.splits - 1) * p.kv_per_split >= p.kv_blocks) --p.splits;
  p.o = o;
  if (p.splits > 1) {
    const size_t rows = static_cast<size_t>(p.splits) * batch * nq;
    p.part_o = partials;
    p.part_m = partials + rows * dv;
    p.part_l = p.part_m + rows;
  }
  (void)part_floats;
  p.status = device_status_word(s);
  if (!p.status) return fail("ib_attention: cannot allocate the device status word");
  p.prof = g_attention_profile;

  const int d_chunks = static_cast<int>((d + 31) / 32);
  const int q_bytes = 2 * d_chunks * kQChunkBytes;
  int ring = (max_smem - 1024 - static_cast<int>(sizeof(Barriers)) - 64 - q_bytes) / kSlotBytes;
  if (ring > kMaxRing) ring = kMaxRing;
  if (ring < 3) return fail("ib_attention: not enough shared memory for the K/V ring");
  p.ring = ring;
  const int smem_bytes = 1024 + q_bytes + ring * kSlotBytes + static_cast<int>(sizeof(Barriers)) + 64;

  CUtensorMap map_q, map_k, map_vt;
  if (int rc = make_tensor_map_f32(&map_q, q, batch, nq, d, d, nq * d, kBQ)) return rc;
  if (int rc = make_tensor_map_f32(&map_k, k, batch, nk, d, d, nk * d, kBKV)) return rc;
  if (int rc = make_tensor_map_f32(&map_vt, vt, batch, dv, nk, nk_pitch, dv * nk_pitch, 128))
    return rc;

  const size_t grid = static_cast<size_t>(p.q_blocks) * p.splits * batch;
  if (grid >= (1u << 31)) return fail("ib_attention: too many work units");
  attention_tf32_kernel<<<static_cast<unsigned>(grid), kThreads, smem_bytes, s>>>(map_q, map_k,
                                                                                 map_vt, p);
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
