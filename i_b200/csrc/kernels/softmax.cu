// Fused row softmax: the reference's three naive kernels
// (ilang-python/flash-attn.py:60-62 — `>ij~i`, `ij-i~ij`, `^ij~ij`, `+ij~i`,
// `ij/i~ij`) collapsed into one pass that keeps the row on chip.
//
// Per row: m = max_c x; e_c = powf(2.71828175f, x_c - m); l = sum_c e_c;
// y_c = e_c / l.  The reference moves 8 matrix-sized streams through memory for
// this chain (two full intermediates); here the row is read once into
// registers and written once, so the algorithmic traffic is 2*rows*cols*4 bytes.
#include "common.cuh"
#include "sm100.cuh"

namespace ib {
namespace {

constexpr int kThreads = 256;

template <int OP, int TPR, int THREADS = kThreads>
__device__ __forceinline__ float row_fold(float v, float* scratch, int row_in_block) {
  if (TPR < 32) {
    // Several rows per warp (short rows): fold among the TPR lanes of a row only.
#pragma unroll
    for (int d = TPR / 2; d > 0; d >>= 1) v = fold<OP>(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
  }
  v = warp_fold<OP>(v);
  if (TPR == 32) return v;
  // TPR == THREADS: one row per CTA.
  const int warp = threadIdx.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
#pragma unroll
  for (int w = 1; w < THREADS / 32; ++w) r = fold<OP>(r, scratch[w]);
  return r;
}

// Row held in registers: VPT float4 per thread, TPR threads per row, THREADS per CTA.  Register
// use is held to 64 so that 1024 threads stay resident per SM (four CTAs of 256, two of 512): at
// 8192 columns that took the kernel from 5.05 to 5.83 TB/s.
template <int VPT, int TPR, bool VEC, int THREADS>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS)
row_softmax_regs(const float* __restrict__ x, float* __restrict__ y, size_t rows, size_t cols) {
  __shared__ float scratch[THREADS / 32];
  constexpr int kRowsPerBlock = THREADS / TPR;
  const int t = threadIdx.x % TPR;
  const int row_in_block = threadIdx.x / TPR;
  const size_t row_blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  for (size_t rb = blockIdx.x; rb < row_blocks; rb += gridDim.x) {
    const size_t r = rb * kRowsPerBlock + row_in_block;
    const bool live = r < rows;
    const float* xr = x + r * cols;
    float* yr = y + r * cols;
    float v[VPT * 4];
    float m = -CUDART_INF_F;
    if (VEC) {
      const size_t nvec = cols / 4;
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        size_t i = static_cast<size_t>(u) * TPR + t;
        float4 q = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        if (live && i < nvec) q = __ldcs(reinterpret_cast<const float4*>(xr) + i);
        v[4 * u + 0] = q.x; v[4 * u + 1] = q.y; v[4 * u + 2] = q.z; v[4 * u + 3] = q.w;
      }
    } else {
#pragma unroll
      for (int u = 0; u < VPT * 4; ++u) {
        size_t i = static_cast<size_t>(u) * TPR + t;
        v[u] = (live && i < cols) ? xr[i] : -CUDART_INF_F;
      }
    }
#pragma unroll
    for (int u = 0; u < VPT * 4; ++u) m = fmaxf(m, v[u]);
    m = row_fold<IB_OP_MAX, TPR, THREADS>(m, scratch, row_in_block);
    float l = 0.0f;
#pragma unroll
    for (int u = 0; u < VPT * 4; ++u) {
      // Padding lanes hold -inf and contribute exp(-inf) = 0.
      v[u] = exp_e32_fast(v[u] - m);
      l += v[u];
    }
    l = row_fold<IB_OP_ADD, TPR, THREADS>(l, scratch, row_in_block);
    // One reciprocal per row instead of a division per element: within 1 ulp of
    // the reference's e / l.
    const float inv = 1.0f / l;
    if (VEC) {
      const size_t nvec = cols / 4;
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        size_t i = static_cast<size_t>(u) * TPR + t;
        if (live && i < nvec)
          __stcs(reinterpret_cast<float4*>(yr) + i,
                 make_float4(v[4 * u] * inv, v[4 * u + 1] * inv, v[4 * u + 2] * inv,
                             v[4 * u + 3] * inv));
      }
    } else {
#pragma unroll
      for (int u = 0; u < VPT * 4; ++u) {
        size_t i = static_cast<size_t>(u) * TPR + t;
        if (live && i < cols) yr[i] = v[u] * inv;
      }
    }
  }
}

// Rows of 32769 to 262144 columns (a vocabulary's logits): the row is held in the registers of a
// thread-block cluster, CLUSTER CTAs of 1024 threads with 32768 columns each, and the row maximum
// and sum meet through distributed shared memory: every CTA publishes its share in its own shared
// memory, a cluster barrier, every CTA reads all shares.  One read and one write of the row, like
// the single-CTA form.  Every CTA of a cluster walks the same rows, so the barriers always match;
// the shares are double-buffered by row parity, which leaves two barriers per row.
template <int CLUSTER, bool VEC>
__global__ void __launch_bounds__(1024, 1)
row_softmax_cluster(const float* __restrict__ x, float* __restrict__ y, size_t rows, size_t cols) {
  constexpr int kVpt = 8, kT = 1024;
  constexpr size_t kSlice = static_cast<size_t>(kVpt) * 4 * kT;     // columns per CTA
  __shared__ float scratch[kT / 32];
  __shared__ float share[2][2];                                    // [row parity][maximum, sum]
  const uint32_t rank = sm100::cluster_cta_rank();
  const size_t cluster = blockIdx.x / CLUSTER, clusters = gridDim.x / CLUSTER;
  const int t = threadIdx.x;
  // Equal shares of the row, a multiple of four columns (at most kSlice by the caller's choice of
  // CLUSTER), so that no CTA of the cluster sits out a ragged row.
  const size_t share_cols = ((cols + CLUSTER - 1) / CLUSTER + 3) / 4 * 4;
  const size_t c_lo = rank * share_cols;
  const size_t c_hi = c_lo + share_cols < cols ? c_lo + share_cols : cols;
  auto all_shares = [&](int parity, int which, bool take_max) {
    float r = take_max ? -CUDART_INF_F : 0.0f;
#pragma unroll
    for (int p = 0; p < CLUSTER; ++p) {
      float v;
      const uint32_t addr = sm100::cluster_addr_of(sm100::smem_u32(&share[parity][which]), p);
      asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
      r = take_max ? fmaxf(r, v) : r + v;
    }
    return r;
  };
  int parity = 0;
  for (size_t r = cluster; r < rows; r += clusters, parity ^= 1) {
    const float* xr = x + r * cols;
    float* yr = y + r * cols;
    float v[kVpt * 4];
    float m = -CUDART_INF_F;
    if (VEC) {
      const size_t nvec = c_hi / 4, v_lo = c_lo / 4;      // cols % 4 == 0 here, so c_hi % 4 == 0
#pragma unroll
      for (int u = 0; u < kVpt; ++u) {
        const size_t i = v_lo + static_cast<size_t>(u) * kT + t;
        float4 q = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        if (i < nvec) q = __ldcs(reinterpret_cast<const float4*>(xr) + i);
        v[4 * u + 0] = q.x; v[4 * u + 1] = q.y; v[4 * u + 2] = q.z; v[4 * u + 3] = q.w;
      }
    } else {
#pragma unroll
      for (int u = 0; u < kVpt * 4; ++u) {
        const size_t i = c_lo + static_cast<size_t>(u) * kT + t;
        v[u] = i < c_hi ? xr[i] : -CUDART_INF_F;
      }
    }
    // One CTA per SM with the registers full: nothing overlaps the next row's trip to memory
    // unless it is asked for now, into L2.
    if (VEC && r + clusters < rows) {
      const float4* next = reinterpret_cast<const float4*>(xr + clusters * cols);
      const size_t nvec = c_hi / 4, v_lo = c_lo / 4;
#pragma unroll
      for (int u = 0; u < kVpt; ++u) {         // a 128-byte line holds eight vectors: one thread in eight asks
        const size_t i = v_lo + static_cast<size_t>(u) * kT + t;
        if (i < nvec && (t & 7) == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(next + i));
      }
    }
#pragma unroll
    for (int u = 0; u < kVpt * 4; ++u) m = fmaxf(m, v[u]);
    m = row_fold<IB_OP_MAX, kT, kT>(m, scratch, 0);
    if (t == 0) share[parity][0] = m;
    sm100::cluster_sync_all();
    m = all_shares(parity, 0, true);
    float l = 0.0f;
#pragma unroll
    for (int u = 0; u < kVpt * 4; ++u) {
      v[u] = exp_e32_fast(v[u] - m);      // padding holds -inf: exp(-inf) = 0
      l += v[u];
    }
    l = row_fold<IB_OP_ADD, kT, kT>(l, scratch, 0);
    if (t == 0) share[parity][1] = l;
    sm100::cluster_sync_all();
    l = all_shares(parity, 1, false);
    const float inv = 1.0f / l;
    if (VEC) {
      const size_t nvec = c_hi / 4, v_lo = c_lo / 4;
#pragma unroll
      for (int u = 0; u < kVpt; ++u) {
        const size_t i = v_lo + static_cast<size_t>(u) * kT + t;
        if (i < nvec)
          __stcs(reinterpret_cast<float4*>(yr) + i,
                 make_float4(v[4 * u] * inv, v[4 * u + 1] * inv, v[4 * u + 2] * inv, v[4 * u + 3] * inv));
      }
    } else {
#pragma unroll
      for (int u = 0; u < kVpt * 4; ++u) {
        const size_t i = c_lo + static_cast<size_t>(u) * kT + t;
        if (i < c_hi) yr[i] = v[u] * inv;
      }
    }
  }
  // No CTA may leave while another still reads its shares.
  sm100::cluster_sync_all();
}

template <int CLUSTER>
int launch_cluster(const float* x, float* y, size_t rows, size_t cols, cudaStream_t s) {
  const bool vec = cols % 4 == 0 && aligned16(x) && aligned16(y);
  int sms = kNumSMs;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  size_t clusters = static_cast<size_t>(sms) / CLUSTER;
  if (clusters > rows) clusters = rows;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = CLUSTER;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(clusters * CLUSTER));
  cfg.blockDim = dim3(1024);
  cfg.stream = s;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  // Clusters are placed inside one GPC each, so fewer may be resident than SMs / CLUSTER; the
  // clusters walk the rows with a fixed stride, so one that waits for a free place would start
  // its share of the rows only when another has finished all of its own.
  int resident = 0;
  const cudaError_t asked =
      vec ? cudaOccupancyMaxActiveClusters(&resident, row_softmax_cluster<CLUSTER, true>, &cfg)
          : cudaOccupancyMaxActiveClusters(&resident, row_softmax_cluster<CLUSTER, false>, &cfg);
  if (asked != cudaSuccess || resident < 1) {
    cudaGetLastError();
    return 1;
  }
  if (static_cast<size_t>(resident) < clusters) cfg.gridDim = dim3(static_cast<unsigned>(resident) * CLUSTER);
  const cudaError_t err = vec ? cudaLaunchKernelEx(&cfg, row_softmax_cluster<CLUSTER, true>, x, y, rows, cols)
                              : cudaLaunchKernelEx(&cfg, row_softmax_cluster<CLUSTER, false>, x, y, rows, cols);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return 1;                                   // the caller falls back to the streaming form
  }
  count_launch();
  return 0;
}

// Rows too long for registers: three streaming passes, one CTA per row.
__global__ void __launch_bounds__(kThreads)
row_softmax_stream(const float* __restrict__ x, float* __restrict__ y, size_t rows, size_t cols) {
  __shared__ float scratch[kThreads / 32];
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* xr = x + r * cols;
    float* yr = y + r * cols;
    float m = -CUDART_INF_F;
    for (size_t i = threadIdx.x; i < cols; i += kThreads) m = fmaxf(m, xr[i]);
    m = row_fold<IB_OP_MAX, kThreads>(m, scratch, 0);
    float l = 0.0f;
    for (size_t i = threadIdx.x; i < cols; i += kThreads) {
      float e = exp_e32_fast(xr[i] - m);
      yr[i] = e;
      l += e;
    }
    l = row_fold<IB_OP_ADD, kThreads>(l, scratch, 0);
    for (size_t i = threadIdx.x; i < cols; i += kThreads) yr[i] = yr[i] / l;
    __syncthreads();
  }
}

template <int VPT, int TPR, int THREADS = kThreads>
int launch_regs(const float* x, float* y, size_t rows, size_t cols, cudaStream_t s) {
  constexpr int kRowsPerBlock = THREADS / TPR;
  size_t blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  size_t cap = static_cast<size_t>(kNumSMs) * 64;
  int grid = static_cast<int>(blocks < cap ? blocks : cap);
  const bool vec = cols % 4 == 0 && aligned16(x) && aligned16(y);
  if (vec)
    row_softmax_regs<VPT, TPR, true, THREADS><<<grid, THREADS, 0, s>>>(x, y, rows, cols);
  else
    row_softmax_regs<VPT, TPR, false, THREADS><<<grid, THREADS, 0, s>>>(x, y, rows, cols);
  return check_launch("ib_row_softmax");
}

}  // namespace
}  // namespace ib

extern "C" int ib_row_softmax(const float* x, float* y, size_t rows, size_t cols, void* stream) {
  if (rows == 0 || cols == 0) return 0;
  if (!x || !y) return ib::fail("ib_row_softmax: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  using namespace ib;
  // Rows shorter than a warp's 128 columns share a warp, so that every lane holds data.
  if (cols <= 16) return launch_regs<1, 4>(x, y, rows, cols, s);
  if (cols <= 32) return launch_regs<1, 8>(x, y, rows, cols, s);
  if (cols <= 64) return launch_regs<1, 16>(x, y, rows, cols, s);
  if (cols <= 128) return launch_regs<1, 32>(x, y, rows, cols, s);
  if (cols <= 256) return launch_regs<2, 32>(x, y, rows, cols, s);
  if (cols <= 512) return launch_regs<4, 32>(x, y, rows, cols, s);
  if (cols <= 1024) return launch_regs<8, 32>(x, y, rows, cols, s);
  if (cols <= 2048) return launch_regs<2, 256>(x, y, rows, cols, s);
  if (cols <= 4096) return launch_regs<4, 256>(x, y, rows, cols, s);
  if (cols <= 8192) return launch_regs<8, 256>(x, y, rows, cols, s);
  if (cols <= 16384) return launch_regs<8, 512, 512>(x, y, rows, cols, s);
  if (cols <= 32768) return launch_regs<8, 1024, 1024>(x, y, rows, cols, s);
  int clustered = 1;
  if (cols <= 2 * 32768) clustered = launch_cluster<2>(x, y, rows, cols, s);
  else if (cols <= 4 * 32768) clustered = launch_cluster<4>(x, y, rows, cols, s);
  else if (cols <= 8 * 32768) clustered = launch_cluster<8>(x, y, rows, cols, s);
  if (clustered == 0) return 0;
  size_t cap = static_cast<size_t>(kNumSMs) * 8;
  row_softmax_stream<<<static_cast<int>(rows < cap ? rows : cap), kThreads, 0, s>>>(x, y, rows,
                                                                                    cols);
  return check_launch("ib_row_softmax");
}
