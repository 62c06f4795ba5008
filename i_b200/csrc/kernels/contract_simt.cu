// CUDA-core fp32 contraction and layout helpers.
//
// ib::contract_simt is the IB_PRECISION_FP32 arm of ib_contract: shared-memory
// tiled FMA GEMM for problems that are too small or too ragged for the tensor
// path (odd K, tiny tiles such as the 8x16x7 product of ilang-python/test.py:
// 52-56).  It computes C[b][i][j] = sum_k A(b,i,k) B(b,j,k) in fp32, the same
// arithmetic as the reference's loop nest (ilang-python/annotated-flashattn.c:
// 57-89) up to summation order and FMA contraction.
//
// ib::transpose_batched rewrites [b][r][c] as [b][c][r]; the tensor path uses
// it to give tcgen05 K-major operands.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"
#include "sm100.cuh"

namespace ib {
namespace {

constexpr int kTile = 64;
constexpr int kTileK = 16;

template <bool A_KMAJOR, bool B_KMAJOR>
__global__ void __launch_bounds__(256)
contract_simt_kernel(const float* __restrict__ a, const float* __restrict__ b,
                     float* __restrict__ c, size_t m, size_t n, size_t k, size_t splits, size_t k_len) {
  __shared__ float sa[kTileK][kTile + 1];
  __shared__ float sb[kTileK][kTile + 1];
  // blockIdx.z = batch entry * splits + split: a split sums k_len terms of the contraction into
  // its own copy of the result (the caller adds the copies).
  const size_t batch = blockIdx.z / splits, split = blockIdx.z - batch * splits;
  a += batch * m * k;
  b += batch * n * k;
  c += static_cast<size_t>(blockIdx.z) * m * n;
  const size_t k_lo = split * k_len, k_hi = k_lo + k_len < k ? k_lo + k_len : k;
  const size_t i0 = static_cast<size_t>(blockIdx.y) * kTile;
  const size_t j0 = static_cast<size_t>(blockIdx.x) * kTile;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (size_t k0 = k_lo; k0 < k_hi; k0 += kTileK) {
    for (int e = threadIdx.x; e < kTile * kTileK; e += 256) {
      // Walk the operand along its contiguous axis.
      int row, kk;
      if (A_KMAJOR) { row = e / kTileK; kk = e % kTileK; } else { kk = e / kTile; row = e % kTile; }
      size_t gi = i0 + row, gk = k0 + kk;
      float v = 0.0f;
      if (gi < m && gk < k_hi) v = A_KMAJOR ? a[gi * k + gk] : a[gk * m + gi];
      sa[kk][row] = v;
      if (B_KMAJOR) { row = e / kTileK; kk = e % kTileK; } else { kk = e / kTile; row = e % kTile; }
      size_t gj = j0 + row;
      gk = k0 + kk;
      v = 0.0f;
      if (gj < n && gk < k_hi) v = B_KMAJOR ? b[gj * k + gk] : b[gk * n + gj];
      sb[kk][row] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        av[u] = sa[kk][ty * 4 + u];
        bv[u] = sb[kk][tx * 4 + u];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int w = 0; w < 4; ++w) acc[u][w] = fmaf(av[u], bv[w], acc[u][w]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    size_t gi = i0 + ty * 4 + u;
    if (gi >= m) continue;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      size_t gj = j0 + tx * 4 + w;
      if (gj < n) c[gi * n + gj] = acc[u][w];
    }
  }
}

// Round-to-nearest fp32 -> tf32 (10-bit mantissa, low 13 bits cleared).  The
// tensor core itself truncates; rounding operands first halves the error and
// removes its bias.
__device__ __forceinline__ float round_tf32(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}

// out[c][r] = in[r][c] through a 64 x 64 tile in shared memory.  Whole tiles of 16-byte-aligned
// arrays move as 16-byte accesses on both sides (a thread loads four neighbouring columns of a row
// and stores four neighbouring rows of a column); ragged or unaligned tiles go element by element.
template <bool ROUND>
__global__ void __launch_bounds__(256)
transpose_kernel(const float* __restrict__ in, float* __restrict__ out, size_t rows, size_t cols,
                 size_t out_pitch, bool vec) {
  constexpr int kT = 64;
  __shared__ float tile[kT][kT + 1];
  const size_t batch = blockIdx.z;
  in += batch * rows * cols;
  out += batch * cols * out_pitch;
  const size_t c0 = static_cast<size_t>(blockIdx.x) * kT, r0 = static_cast<size_t>(blockIdx.y) * kT;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const bool whole = vec && r0 + kT <= rows && c0 + kT <= cols;
  if (whole) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int r = ty + 16 * p;
      const float4 v = *reinterpret_cast<const float4*>(in + (r0 + r) * cols + c0 + 4 * tx);
      tile[r][4 * tx + 0] = v.x;
      tile[r][4 * tx + 1] = v.y;
      tile[r][4 * tx + 2] = v.z;
      tile[r][4 * tx + 3] = v.w;
    }
  } else {
    for (int e = threadIdx.x; e < kT * kT; e += 256) {
      const int r = e / kT, c = e % kT;
      if (r0 + r < rows && c0 + c < cols) tile[r][c] = in[(r0 + r) * cols + c0 + c];
    }
  }
  __syncthreads();
  if (whole) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int c = ty + 16 * p;
      float4 v = make_float4(tile[4 * tx + 0][c], tile[4 * tx + 1][c], tile[4 * tx + 2][c], tile[4 * tx + 3][c]);
      if (ROUND) v = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
      *reinterpret_cast<float4*>(out + (c0 + c) * out_pitch + r0 + 4 * tx) = v;
    }
  } else {
    for (int e = threadIdx.x; e < kT * kT; e += 256) {
      const int c = e / kT, r = e % kT;
      if (r0 + r < rows && c0 + c < cols)
        out[(c0 + c) * out_pitch + r0 + r] = ROUND ? round_tf32(tile[r][c]) : tile[r][c];
    }
  }
}

// out[r][c] = round_tf32(in[r][c]) for up to two row-major arrays in one launch
// (blockIdx.y selects the array); pitches in elements.
struct RoundJob {
  const float* in;
  float* out;
  size_t rows, cols, in_pitch, out_pitch;
};

__global__ void __launch_bounds__(256)
round_rows_kernel(RoundJob j0, RoundJob j1) {
  const RoundJob j = blockIdx.y == 0 ? j0 : j1;
  const size_t n = j.rows * j.cols;
  const size_t stride = static_cast<size_t>(gridDim.x) * 256;
  const bool vec = j.cols % 4 == 0 && j.in_pitch % 4 == 0 && j.out_pitch % 4 == 0 &&
                   (reinterpret_cast<uintptr_t>(j.in) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(j.out) & 15u) == 0;
  if (vec) {
    const size_t cvec = j.cols / 4;
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < n / 4; i += stride) {
      const size_t r = i / cvec, c = (i - r * cvec) * 4;
      float4 v = *reinterpret_cast<const float4*>(j.in + r * j.in_pitch + c);
      v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w);
      *reinterpret_cast<float4*>(j.out + r * j.out_pitch + c) = v;
    }
  } else {
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < n; i += stride) {
      const size_t r = i / j.cols, c = i - r * j.cols;
      j.out[r * j.out_pitch + c] = round_tf32(j.in[r * j.in_pitch + c]);
    }
  }
}

// Operand preparation for the fused attention kernel in one launch:
// blockIdx.y = 0 rounds Q, 1 rounds K (both plain copies with TF32 rounding),
// 2 writes V^T = round(V)^T with 64x64 tiles through shared memory.
struct PrepareArgs {
  const float* q; float* qr; size_t q_elems;
  const float* k; float* kr; size_t k_elems;
  const float* v; float* vt; size_t batch, nk, dv, pitch;
};

__global__ void __launch_bounds__(256)
prepare_attention_kernel(PrepareArgs a) {
  __shared__ float tile[64][65];
  // The attention kernel may be scheduled once every CTA of this grid has started;
  // it waits for this grid's completion before it reads K or V^T.
  sm100::trigger_dependent_launch();
  if (blockIdx.y < 2) {
    const float* in = blockIdx.y == 0 ? a.q : a.k;
    float* out = blockIdx.y == 0 ? a.qr : a.kr;
    const size_t n4 = (blockIdx.y == 0 ? a.q_elems : a.k_elems) / 4;   // element counts are multiples of 4
    const size_t stride = static_cast<size_t>(gridDim.x) * 256;
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < n4; i += stride) {
      float4 x = __ldcs(reinterpret_cast<const float4*>(in) + i);
      x.x = round_tf32(x.x); x.y = round_tf32(x.y); x.z = round_tf32(x.z); x.w = round_tf32(x.w);
      reinterpret_cast<float4*>(out)[i] = x;
    }
    return;
  }
  const size_t tiles_k = (a.nk + 63) / 64, tiles_d = (a.dv + 63) / 64;
  const size_t total = a.batch * tiles_k * tiles_d;
  const bool vec_in = a.dv % 4 == 0 && (reinterpret_cast<uintptr_t>(a.v) & 15u) == 0;
  const bool vec_out = a.pitch % 4 == 0 && (reinterpret_cast<uintptr_t>(a.vt) & 15u) == 0;
  for (size_t t = blockIdx.x; t < total; t += gridDim.x) {
    const size_t b = t / (tiles_k * tiles_d);
    const size_t rem = t - b * tiles_k * tiles_d;
    const size_t k0 = (rem / tiles_d) * 64, d0 = (rem % tiles_d) * 64;
    const float* src = a.v + b * a.nk * a.dv;
    float* dst = a.vt + b * a.dv * a.pitch;
    // 64 keys x 64 features in: 16 float4 per key row, 4 rows per thread.
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int r = e >> 4, c = (e & 15) * 4;           // r: key, c: feature (contiguous in V)
      float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (k0 + r < a.nk) {
        const float* row = src + (k0 + r) * a.dv + d0 + c;
        if (vec_in && d0 + c + 4 <= a.dv) {
          x = __ldcs(reinterpret_cast<const float4*>(row));
        } else {
          if (d0 + c + 0 < a.dv) x.x = row[0];
          if (d0 + c + 1 < a.dv) x.y = row[1];
          if (d0 + c + 2 < a.dv) x.z = row[2];
          if (d0 + c + 3 < a.dv) x.w = row[3];
        }
      }
      tile[r][c + 0] = round_tf32(x.x);
      tile[r][c + 1] = round_tf32(x.y);
      tile[r][c + 2] = round_tf32(x.z);
      tile[r][c + 3] = round_tf32(x.w);
    }
    __syncthreads();
    // 64 features x 64 keys out: 16 float4 per feature row.
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int c = e >> 4, r = (e & 15) * 4;           // c: feature, r: key (contiguous in V^T)
      if (d0 + c >= a.dv) continue;
      float* row = dst + (d0 + c) * a.pitch + k0 + r;
      const float4 x = make_float4(tile[r][c], tile[r + 1][c], tile[r + 2][c], tile[r + 3][c]);
      if (vec_out && k0 + r + 4 <= a.nk) {
        *reinterpret_cast<float4*>(row) = x;
      } else {
        if (k0 + r + 0 < a.nk) row[0] = x.x;
        if (k0 + r + 1 < a.nk) row[1] = x.y;
        if (k0 + r + 2 < a.nk) row[2] = x.z;
        if (k0 + r + 3 < a.nk) row[3] = x.w;
      }
    }
    __syncthreads();
  }
}

__device__ __forceinline__ uint2 pack4_bf16(float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

__global__ void __launch_bounds__(256)
convert_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t rows,
                    size_t cols, size_t out_pitch) {
  // Four output columns per thread: a 16-byte load and an 8-byte store (out_pitch is a
  // multiple of 8, so every row starts 16-byte aligned).
  const size_t quads = out_pitch / 4;
  const size_t total = rows * quads;
  const size_t stride = static_cast<size_t>(gridDim.x) * 256;
  const bool vec = cols % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
  for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += stride) {
    const size_t r = i / quads, c = (i - r * quads) * 4;
    float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float* src = in + r * cols + c;
    if (vec && c + 4 <= cols) {
      x = __ldcs(reinterpret_cast<const float4*>(src));
    } else {
      if (c + 0 < cols) x.x = src[0];
      if (c + 1 < cols) x.y = src[1];
      if (c + 2 < cols) x.z = src[2];
      if (c + 3 < cols) x.w = src[3];
    }
    *reinterpret_cast<uint2*>(out + r * out_pitch + c) = pack4_bf16(x.x, x.y, x.z, x.w);
  }
}

// bf16 operand preparation for attention, one launch: blockIdx.y = 0 converts K
// ([rows][d] -> [rows][d_pitch]), blockIdx.y = 1 writes V^T ([nk][dv] -> [dv][nk_pitch])
// through 64x64 shared-memory tiles.  Pad columns are written as zero.
struct PrepareBf16Args {
  const float* k; __nv_bfloat16* k16; size_t k_rows, d, d_pitch;
  const float* v; __nv_bfloat16* vt16; size_t batch, nk, dv, nk_pitch;
};

__global__ void __launch_bounds__(256)
prepare_attention_bf16_kernel(PrepareBf16Args a) {
  __shared__ float tile[64][65];
  sm100::trigger_dependent_launch();       // see prepare_attention_kernel
  if (blockIdx.y == 0) {
    // Four columns per thread: one 16-byte load, one 8-byte store (d_pitch is a multiple of 8).
    const size_t quads = a.d_pitch / 4, total = a.k_rows * quads;
    const size_t stride = static_cast<size_t>(gridDim.x) * 256;
    const bool vec = a.d % 4 == 0 && (reinterpret_cast<uintptr_t>(a.k) & 15u) == 0;
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += stride) {
      const size_t r = i / quads, c = (i - r * quads) * 4;
      float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      const float* src = a.k + r * a.d + c;
      if (vec && c + 4 <= a.d) {
        x = __ldcs(reinterpret_cast<const float4*>(src));
      } else {
        if (c + 0 < a.d) x.x = src[0];
        if (c + 1 < a.d) x.y = src[1];
        if (c + 2 < a.d) x.z = src[2];
        if (c + 3 < a.d) x.w = src[3];
      }
      *reinterpret_cast<uint2*>(a.k16 + r * a.d_pitch + c) = pack4_bf16(x.x, x.y, x.z, x.w);
    }
    return;
  }
  const size_t tiles_k = (a.nk_pitch + 63) / 64, tiles_d = (a.dv + 63) / 64;
  const size_t total = a.batch * tiles_k * tiles_d;
  const bool vec_in = a.dv % 4 == 0 && (reinterpret_cast<uintptr_t>(a.v) & 15u) == 0;
  for (size_t t = blockIdx.x; t < total; t += gridDim.x) {
    const size_t b = t / (tiles_k * tiles_d);
    const size_t rem = t - b * tiles_k * tiles_d;
    const size_t k0 = (rem / tiles_d) * 64, d0 = (rem % tiles_d) * 64;
    const float* src = a.v + b * a.nk * a.dv;
    __nv_bfloat16* dst = a.vt16 + b * a.dv * a.nk_pitch;
    // 64 keys x 64 features in: 16 float4 per key row.
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int r = e >> 4, c = (e & 15) * 4;           // r: key, c: feature (contiguous in V)
      float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (k0 + r < a.nk) {
        const float* row = src + (k0 + r) * a.dv + d0 + c;
        if (vec_in && d0 + c + 4 <= a.dv) {
          x = __ldcs(reinterpret_cast<const float4*>(row));
        } else {
          if (d0 + c + 0 < a.dv) x.x = row[0];
          if (d0 + c + 1 < a.dv) x.y = row[1];
          if (d0 + c + 2 < a.dv) x.z = row[2];
          if (d0 + c + 3 < a.dv) x.w = row[3];
        }
      }
      tile[r][c + 0] = x.x; tile[r][c + 1] = x.y; tile[r][c + 2] = x.z; tile[r][c + 3] = x.w;
    }
    __syncthreads();
    // 64 features x 64 keys out: 16 groups of 4 keys (8 bytes) per feature row; keys past nk
    // (up to the pitch) are written as the zeros the load left in the tile.
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int c = e >> 4, r = (e & 15) * 4;           // c: feature, r: first key of the group
      if (d0 + c < a.dv && k0 + r < a.nk_pitch)
        *reinterpret_cast<uint2*>(dst + (d0 + c) * a.nk_pitch + k0 + r) =
            pack4_bf16(tile[r][c], tile[r + 1][c], tile[r + 2][c], tile[r + 3][c]);
    }
    __syncthreads();
  }
}

// ---- mixed arm: K rounded to TF32, V^T as fp16 scaled per head into fp16's range ----

// Largest |v| of each head, in kAbsmaxBlocks partial maxima per head (no atomics).  gridDim.y <=
// kAbsmaxBlocks blocks share a head, each thread keeping eight 16-byte loads in flight; the slots of
// the blocks a short head does not need are written as zero by its first block.
__global__ void __launch_bounds__(256)
absmax_heads_kernel(const float* __restrict__ v, float* __restrict__ block_max, size_t per_head) {
  __shared__ float warp_max[8];
  // The conversion kernel behind this one may start now: its K half does not need these maxima,
  // its V half waits for this grid before it reads them.
  sm100::trigger_dependent_launch();
  // blockIdx.x = head, blockIdx.y = slice of the head
  const float* base = v + static_cast<size_t>(blockIdx.x) * per_head;
  float m = 0.0f;
  const bool vec = per_head % 4 == 0 && (reinterpret_cast<uintptr_t>(base) & 15u) == 0;
  const size_t stride = static_cast<size_t>(gridDim.y) * 256;
  if (vec) {
    const float4* b4 = reinterpret_cast<const float4*>(base);
    const size_t n4 = per_head / 4;
    for (size_t i0 = static_cast<size_t>(blockIdx.y) * 256 + threadIdx.x; i0 < n4; i0 += 8 * stride) {
      float4 x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)   // plain loads: the conversion pass reads V again
        x[u] = i0 + u * stride < n4 ? b4[i0 + u * stride] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        m = fmaxf(m, fmaxf(fmaxf(fabsf(x[u].x), fabsf(x[u].y)), fmaxf(fabsf(x[u].z), fabsf(x[u].w))));
    }
  } else {
    for (size_t i = static_cast<size_t>(blockIdx.y) * 256 + threadIdx.x; i < per_head; i += stride)
      m = fmaxf(m, fabsf(base[i]));
  }
  m = warp_fold<IB_OP_MAX>(m);
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  float* slots = block_max + static_cast<size_t>(blockIdx.x) * kAbsmaxBlocks;
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w]);
    slots[blockIdx.y] = m;
  }
  if (blockIdx.y == 0)
    for (int i = gridDim.y + threadIdx.x; i < kAbsmaxBlocks; i += 256) slots[i] = 0.0f;
}

// The power of two that brings a head's largest magnitude into [2^14, 2^15): large values fit
// fp16 (which holds up to 65504) and small ones keep their mantissa instead of falling into
// fp16's subnormals.  1 for an all-zero head or one holding inf / NaN (which then propagate as
// they would anyway).
__device__ __forceinline__ float f16_scale_for(float absmax) {
  if (!(absmax > 0.0f) || !(absmax < CUDART_INF_F)) return 1.0f;
  int e;
  frexpf(absmax, &e);                          // absmax = f * 2^e, f in [0.5, 1)
  return ldexpf(1.0f, max(e - 15, -120));      // absmax / scale = f * 2^15
}

// Every thread returns the scale of head b (reduces that head's partial maxima).
__device__ __forceinline__ float head_scale(const float* block_max, size_t b, float* scratch) {
  float m = threadIdx.x < kAbsmaxBlocks ? block_max[b * kAbsmaxBlocks + threadIdx.x] : 0.0f;
  m = warp_fold<IB_OP_MAX>(m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
  __syncthreads();
  float all = scratch[0];
  for (int w = 1; w < 8; ++w) all = fmaxf(all, scratch[w]);
  return f16_scale_for(all);
}

__device__ __forceinline__ uint2 pack4_f16(float a, float b, float c, float d) {
  const __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
  return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

struct PrepareMixedArgs {
  const float* k; float* kr; size_t k_elems;
  const float* v; __half* vt16; float* scale; const float* block_max;
  size_t batch, nk, dv, nk_pitch;
  int v_kmajor;
  // fp16 arm only: K as fp16 [batch][nk][d_pitch], each tile of 128 keys over its own power of two.
  __half* k16; float* k_tile_scale; size_t d, d_pitch, kv_tiles;
};

// fp16(V^T / scale[head]) — through shared memory in steps of 64 keys when V is [keys][dv], as plain
// rows when it is already [dv][keys].  The per-head maxima come from the kernel before this one.
__device__ __forceinline__ void prepare_v_f16(const PrepareMixedArgs& a, uint32_t (*words)[32],
                                              float* scratch) {
  sm100::grid_dependency_wait();
  if (a.v_kmajor) {
    // Rows [batch * dv][nk] -> [batch * dv][nk_pitch], one row per block at a time.
    const size_t quads = a.nk_pitch / 4;
    const bool vec = a.nk % 4 == 0 && (reinterpret_cast<uintptr_t>(a.v) & 15u) == 0;
    size_t scaled_for = static_cast<size_t>(-1);
    float inv = 1.0f;
    for (size_t row = blockIdx.x; row < a.batch * a.dv; row += gridDim.x) {
      const size_t b = row / a.dv;
      if (b != scaled_for) {
        inv = 1.0f / head_scale(a.block_max, b, scratch);
        scaled_for = b;
      }
      if (row == b * a.dv && threadIdx.x == 0) a.scale[b] = 1.0f / inv;
      for (size_t q = threadIdx.x; q < quads; q += 256) {
        const size_t c = q * 4;
        const float* src = a.v + row * a.nk + c;
        float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (vec && c + 4 <= a.nk) {
          x = __ldcs(reinterpret_cast<const float4*>(src));
        } else {
          if (c + 0 < a.nk) x.x = src[0];
          if (c + 1 < a.nk) x.y = src[1];
          if (c + 2 < a.nk) x.z = src[2];
          if (c + 3 < a.nk) x.w = src[3];
        }
        *reinterpret_cast<uint2*>(a.vt16 + row * a.nk_pitch + c) =
            pack4_f16(x.x * inv, x.y * inv, x.z * inv, x.w * inv);
      }
    }
    return;
  }
  // 64 keys x all dv features per step.  Warp w takes key pairs 4w .. 4w + 3 of the step; lane l
  // loads features 4l .. 4l + 3 of both keys of a pair (two coalesced 512-byte rows), so eight
  // 16-byte loads are in flight per thread.  A pair of keys of one feature is one fp16x2 word of
  // V^T; it goes through shared memory as word [feature][pair ^ (feature / 4)]: the 32 lanes of a
  // store (32 feature groups, one pair) and the 32 lanes of a read (one feature, 32 pairs) each
  // hit 32 different banks.  A warp then writes a feature's 64 keys as one 128-byte line.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t tiles_k = (a.nk_pitch + 63) / 64;
  const size_t total = a.batch * tiles_k;
  const bool vec_in = a.dv % 4 == 0 && (reinterpret_cast<uintptr_t>(a.v) & 15u) == 0;
  size_t scaled_for = static_cast<size_t>(-1);
  float inv = 1.0f;
  for (size_t t = blockIdx.x; t < total; t += gridDim.x) {
    const size_t b = t / tiles_k;
    const size_t k0 = (t - b * tiles_k) * 64;
    if (b != scaled_for) {
      inv = 1.0f / head_scale(a.block_max, b, scratch);
      scaled_for = b;
    }
    if (k0 == 0 && threadIdx.x == 0) a.scale[b] = 1.0f / inv;   // the block with the head's first tile
    const float* src = a.v + b * a.nk * a.dv;
    __half* dst = a.vt16 + b * a.dv * a.nk_pitch;
    const int c = lane * 4;                               // first feature of this lane's group
    float4 x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const size_t key = k0 + static_cast<size_t>(2 * (warp * 4 + (u >> 1)) + (u & 1));
      x[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (key < a.nk && static_cast<size_t>(c) < a.dv) {
        const float* row = src + key * a.dv + c;
        if (vec_in && static_cast<size_t>(c) + 4 <= a.dv) {
          x[u] = __ldcs(reinterpret_cast<const float4*>(row));
        } else {
          x[u].x = row[0];
          if (static_cast<size_t>(c) + 1 < a.dv) x[u].y = row[1];
          if (static_cast<size_t>(c) + 2 < a.dv) x[u].z = row[2];
          if (static_cast<size_t>(c) + 3 < a.dv) x[u].w = row[3];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; u += 2) {
      const int pair = warp * 4 + (u >> 1);
      const int col = pair ^ lane;                        // (feature / 4) & 31 == lane for all four
      const __half2 w0 = __floats2half2_rn(x[u].x * inv, x[u + 1].x * inv);
      const __half2 w1 = __floats2half2_rn(x[u].y * inv, x[u + 1].y * inv);
      const __half2 w2 = __floats2half2_rn(x[u].z * inv, x[u + 1].z * inv);
      const __half2 w3 = __floats2half2_rn(x[u].w * inv, x[u + 1].w * inv);
      words[c + 0][col] = *reinterpret_cast<const uint32_t*>(&w0);
      words[c + 1][col] = *reinterpret_cast<const uint32_t*>(&w1);
      words[c + 2][col] = *reinterpret_cast<const uint32_t*>(&w2);
      words[c + 3][col] = *reinterpret_cast<const uint32_t*>(&w3);
    }
    __syncthreads();
    // Feature rows warp, warp + 8, ...: lane = key pair.  Keys past nk (up to the pitch, which is
    // even) are written as the zeros the loads left.
#pragma unroll 4
    for (int f = warp; f < 128; f += 8) {
      if (static_cast<size_t>(f) < a.dv && k0 + 2 * lane < a.nk_pitch)
        *reinterpret_cast<uint32_t*>(dst + static_cast<size_t>(f) * a.nk_pitch + k0 + 2 * lane) =
            words[f][lane ^ ((f >> 2) & 31)];
    }
    __syncthreads();
  }
}

// The same in steps of 64 keys x 64 features (53 registers: for the grid whose other half is a plain
// elementwise pass and lives on occupancy).  fp16(V^T / scale[head]) — through 64x64 shared-memory tiles when V is [keys][dv], as plain rows
// when it is already [dv][keys].  The per-head maxima come from the kernel before this one.
__device__ __forceinline__ void prepare_v_f16_by_quarters(const PrepareMixedArgs& a, float (*tile)[65],
                                              float* scratch) {
  sm100::grid_dependency_wait();
  if (a.v_kmajor) {
    // Rows [batch * dv][nk] -> [batch * dv][nk_pitch], one row per block at a time.
    const size_t quads = a.nk_pitch / 4;
    const bool vec = a.nk % 4 == 0 && (reinterpret_cast<uintptr_t>(a.v) & 15u) == 0;
    size_t scaled_for = static_cast<size_t>(-1);
    float inv = 1.0f;
    for (size_t row = blockIdx.x; row < a.batch * a.dv; row += gridDim.x) {
      const size_t b = row / a.dv;
      if (b != scaled_for) {
        inv = 1.0f / head_scale(a.block_max, b, scratch);
        scaled_for = b;
      }
      if (row == b * a.dv && threadIdx.x == 0) a.scale[b] = 1.0f / inv;
      for (size_t q = threadIdx.x; q < quads; q += 256) {
        const size_t c = q * 4;
        const float* src = a.v + row * a.nk + c;
        float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (vec && c + 4 <= a.nk) {
          x = __ldcs(reinterpret_cast<const float4*>(src));
        } else {
          if (c + 0 < a.nk) x.x = src[0];
          if (c + 1 < a.nk) x.y = src[1];
          if (c + 2 < a.nk) x.z = src[2];
          if (c + 3 < a.nk) x.w = src[3];
        }
        *reinterpret_cast<uint2*>(a.vt16 + row * a.nk_pitch + c) =
            pack4_f16(x.x * inv, x.y * inv, x.z * inv, x.w * inv);
      }
    }
    return;
  }
  const size_t tiles_k = (a.nk_pitch + 63) / 64, tiles_d = (a.dv + 63) / 64;
  const size_t total = a.batch * tiles_k * tiles_d;
  const bool vec_in = a.dv % 4 == 0 && (reinterpret_cast<uintptr_t>(a.v) & 15u) == 0;
  size_t scaled_for = static_cast<size_t>(-1);
  float inv = 1.0f;
  for (size_t t = blockIdx.x; t < total; t += gridDim.x) {
    const size_t b = t / (tiles_k * tiles_d);
    const size_t rem = t - b * tiles_k * tiles_d;
    if (b != scaled_for) {
      inv = 1.0f / head_scale(a.block_max, b, scratch);
      scaled_for = b;
    }
    if (rem == 0 && threadIdx.x == 0) a.scale[b] = 1.0f / inv;   // the block with the head's first tile
    const size_t k0 = (rem / tiles_d) * 64, d0 = (rem % tiles_d) * 64;
    const float* src = a.v + b * a.nk * a.dv;
    __half* dst = a.vt16 + b * a.dv * a.nk_pitch;
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int r = e >> 4, c = (e & 15) * 4;           // r: key, c: feature (contiguous in V)
      float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (k0 + r < a.nk) {
        const float* row = src + (k0 + r) * a.dv + d0 + c;
        if (vec_in && d0 + c + 4 <= a.dv) {
          x = __ldcs(reinterpret_cast<const float4*>(row));
        } else {
          if (d0 + c + 0 < a.dv) x.x = row[0];
          if (d0 + c + 1 < a.dv) x.y = row[1];
          if (d0 + c + 2 < a.dv) x.z = row[2];
          if (d0 + c + 3 < a.dv) x.w = row[3];
        }
      }
      tile[r][c + 0] = x.x * inv; tile[r][c + 1] = x.y * inv;
      tile[r][c + 2] = x.z * inv; tile[r][c + 3] = x.w * inv;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int c = e >> 4, r = (e & 15) * 4;           // c: feature, r: first key of the group
      if (d0 + c < a.dv && k0 + r < a.nk_pitch)
        *reinterpret_cast<uint2*>(dst + (d0 + c) * a.nk_pitch + k0 + r) =
            pack4_f16(tile[r][c], tile[r + 1][c], tile[r + 2][c], tile[r + 3][c]);
    }
    __syncthreads();
  }
}

// blockIdx.y = 0 rounds K to TF32; blockIdx.y = 1 writes the fp16 V^T.
__global__ void __launch_bounds__(256)
prepare_attention_mixed_kernel(PrepareMixedArgs a) {
  __shared__ float tile[64][65];
  __shared__ float scratch[8];
  sm100::trigger_dependent_launch();       // see prepare_attention_kernel
  if (blockIdx.y == 0) {
    const size_t n4 = a.k_elems / 4;          // d is a multiple of 4
    const size_t stride = static_cast<size_t>(gridDim.x) * 256;
    const bool vec = (reinterpret_cast<uintptr_t>(a.k) & 15u) == 0;
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < n4; i += stride) {
      float4 x;
      if (vec) {
        x = __ldcs(reinterpret_cast<const float4*>(a.k) + i);
      } else {
        x = make_float4(a.k[4 * i], a.k[4 * i + 1], a.k[4 * i + 2], a.k[4 * i + 3]);
      }
      x.x = round_tf32(x.x); x.y = round_tf32(x.y); x.z = round_tf32(x.z); x.w = round_tf32(x.w);
      reinterpret_cast<float4*>(a.kr)[i] = x;
    }
    return;
  }
  prepare_v_f16_by_quarters(a, tile, scratch);
}

// fp16 arm.  blockIdx.y = 0: K, one tile of 128 keys per block at a time: the tile is read once
// twice (the second time from cache), its largest magnitude decides the power of two that brings it into
// [2^14, 2^15), and fp16(K / that) is written with rows padded to d_pitch (pad columns zero).  An
// outlier key therefore costs precision only to the 127 keys beside it.  blockIdx.y = 1: the fp16
// V^T as in the mixed arm.
template <bool FEW_TILES>
__global__ void __launch_bounds__(256)
prepare_attention_f16_kernel(PrepareMixedArgs a, int halves) {
  __shared__ uint32_t words[128][32];      // a step of V^T: 128 features x 32 key pairs (fp16x2)
  __shared__ float scratch[8];
  sm100::trigger_dependent_launch();       // see prepare_attention_kernel
  // halves: 3 = this grid does both (blockIdx.y picks), 1 = K only, 2 = V only.
  if ((halves == 3 ? blockIdx.y : halves - 1) == 1) {
    prepare_v_f16(a, words, scratch);
    return;
  }
  const size_t quads = a.d_pitch / 4;       // 4-column groups per (padded) key row, at most 32
  const bool vec = (reinterpret_cast<uintptr_t>(a.k) & 15u) == 0;   // d is a multiple of 4
  // With few tiles (one head of a few thousand keys) the blocks are too few to hide two rounds of
  // loads each: a thread then keeps its share of the tile in registers (sixteen 16-byte loads in
  // flight, 118 registers) and the second pass is free.  With many tiles that register count
  // would hold the V half of this grid to two blocks per SM, and eight loads at a time at 64
  // registers is the faster whole.
  constexpr int kBatch = FEW_TILES ? 16 : 8;
  for (size_t t = blockIdx.x; t < a.batch * a.kv_tiles; t += gridDim.x) {
    const size_t b = t / a.kv_tiles, key0 = (t - b * a.kv_tiles) * 128;
    const size_t keys = a.nk - key0 < 128 ? a.nk - key0 : 128;
    const float* src = a.k + (b * a.nk + key0) * a.d;
    __half* dst = a.k16 + (b * a.nk + key0) * a.d_pitch;
    const size_t groups = keys * quads;
    auto fetch = [&](size_t g) {
      const size_t r = g / quads, c = (g - r * quads) * 4;
      if (g >= groups || c >= a.d) return make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      const float* at = src + r * a.d + c;
      return vec ? *reinterpret_cast<const float4*>(at) : make_float4(at[0], at[1], at[2], at[3]);
    };
    // Pass 1: the tile's largest magnitude.  Pass 2 reads the same 64 KB again, from cache, unless
    // the thread's whole share (128 x 32 groups over 256 threads = 16) is still in registers.
    float m = 0.0f;
    float4 x[kBatch];
    for (size_t g0 = threadIdx.x; g0 < groups; g0 += 256 * kBatch) {
#pragma unroll
      for (int u = 0; u < kBatch; ++u) x[u] = fetch(g0 + static_cast<size_t>(u) * 256);
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        m = fmaxf(m, fmaxf(fmaxf(fabsf(x[u].x), fabsf(x[u].y)), fmaxf(fabsf(x[u].z), fabsf(x[u].w))));
    }
    m = warp_fold<IB_OP_MAX>(m);
    __syncthreads();                         // scratch may still be read from the tile before
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
    __syncthreads();
    float all = scratch[0];
    for (int w = 1; w < 8; ++w) all = fmaxf(all, scratch[w]);
    const float scale = f16_scale_for(all);
    const float inv = 1.0f / scale;
    if (threadIdx.x == 0) a.k_tile_scale[t] = scale;
    for (size_t g0 = threadIdx.x; g0 < groups; g0 += 256 * kBatch) {
      if (!FEW_TILES) {
#pragma unroll
        for (int u = 0; u < kBatch; ++u) x[u] = fetch(g0 + static_cast<size_t>(u) * 256);
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const size_t g = g0 + static_cast<size_t>(u) * 256;
        if (g < groups) {
          const size_t r = g / quads, c = (g - r * quads) * 4;
          *reinterpret_cast<uint2*>(dst + r * a.d_pitch + c) =
              pack4_f16(x[u].x * inv, x[u].y * inv, x[u].z * inv, x[u].w * inv);
        }
      }
    }
  }
  // Launched on its own under the tail of the maxima kernel (many tiles): this grid then only
  // completes once that one has, so that whoever waits for this grid has waited for both.
  if (halves == 1) sm100::grid_dependency_wait();
}

// fp16 operand of a contraction: one warp per row.  Pass 1 finds the row's largest magnitude, pass 2
// (the row again, from cache) writes fp16(row / scale) with scale the power of two that brings that
// magnitude into [2^14, 2^15), and the scale itself for the epilogue to multiply back.  Pad columns
// up to the pitch are written as zero.
__global__ void __launch_bounds__(256)
convert_f16_rows_scaled_kernel(const float* __restrict__ in, __half* __restrict__ out,
                               float* __restrict__ scale_out, size_t rows, size_t cols,
                               size_t out_pitch) {
  const int lane = threadIdx.x & 31;
  const size_t warps_total = static_cast<size_t>(gridDim.x) * 8;
  const bool vec = cols % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
  const size_t quads = out_pitch / 4;
  for (size_t r = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); r < rows;
       r += warps_total) {
    const float* src = in + r * cols;
    auto fetch = [&](size_t q) {
      const size_t c = q * 4;
      float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (vec && c + 4 <= cols) {
        x = *reinterpret_cast<const float4*>(src + c);
      } else {
        if (c + 0 < cols) x.x = src[c + 0];
        if (c + 1 < cols) x.y = src[c + 1];
        if (c + 2 < cols) x.z = src[c + 2];
        if (c + 3 < cols) x.w = src[c + 3];
      }
      return x;
    };
    float m = 0.0f;
    for (size_t q0 = lane; q0 < quads; q0 += 32 * 8) {
      float4 x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        x[u] = q0 + u * 32 < quads ? fetch(q0 + u * 32) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        m = fmaxf(m, fmaxf(fmaxf(fabsf(x[u].x), fabsf(x[u].y)), fmaxf(fabsf(x[u].z), fabsf(x[u].w))));
    }
    m = warp_fold<IB_OP_MAX>(m);
    const float scale = f16_scale_for(m);
    const float inv = 1.0f / scale;
    if (lane == 0) scale_out[r] = scale;
    __half* dst = out + r * out_pitch;
    for (size_t q0 = lane; q0 < quads; q0 += 32 * 8) {
      float4 x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        x[u] = q0 + u * 32 < quads ? fetch(q0 + u * 32) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (q0 + u * 32 < quads)
          *reinterpret_cast<uint2*>(dst + (q0 + u * 32) * 4) =
              pack4_f16(x[u].x * inv, x[u].y * inv, x[u].z * inv, x[u].w * inv);
    }
  }
}

}  // namespace

// Blocks that share a head in absmax_heads_kernel: one per 32 KB of the head (eight 16-byte loads
// per thread), at most kAbsmaxBlocks.
unsigned absmax_blocks_per_head(size_t per_head) {
  const size_t per_block = 256 * 4 * 8;
  size_t blocks = (per_head + per_block - 1) / per_block;
  if (blocks < 1) blocks = 1;
  if (blocks > static_cast<size_t>(kAbsmaxBlocks)) blocks = kAbsmaxBlocks;
  return static_cast<unsigned>(blocks);
}

int prepare_attention_operands_bf16(const float* k, void* k16, const float* v, void* vt16,
                                    size_t batch, size_t nk, size_t d, size_t dv, size_t d_pitch,
                                    size_t nk_pitch, bool v_kmajor, cudaStream_t s) {
  if (v_kmajor) {
    // V already [dv][nk]: both operands are plain row conversions.
    if (int rc = convert_bf16_rows(k, k16, batch * nk, d, d_pitch, s)) return rc;
    return convert_bf16_rows(v, vt16, batch * dv, nk, nk_pitch, s);
  }
  PrepareBf16Args a{k, static_cast<__nv_bfloat16*>(k16), batch * nk, d, d_pitch,
                    v, static_cast<__nv_bfloat16*>(vt16), batch, nk, dv, nk_pitch};
  const size_t most = std::max(batch * nk * d_pitch / 4 / 256 + 1,
                               batch * ((nk_pitch + 63) / 64) * ((dv + 63) / 64));
  const size_t cap = static_cast<size_t>(kNumSMs) * 8;
  dim3 grid(static_cast<unsigned>(std::min(most, cap)), 2);
  prepare_attention_bf16_kernel<<<grid, 256, 0, s>>>(a);
  return check_launch("prepare_attention_operands_bf16");
}

int prepare_attention_operands_mixed(const float* k, float* kr, const float* v, void* vt16,
                                     float* scale, float* block_max, size_t batch, size_t nk,
                                     size_t d, size_t dv, size_t nk_pitch, bool v_kmajor,
                                     cudaStream_t s) {
  dim3 agrid(static_cast<unsigned>(batch), absmax_blocks_per_head(nk * dv));
  absmax_heads_kernel<<<agrid, 256, 0, s>>>(v, block_max, nk * dv);
  if (int rc = check_launch("absmax_heads")) return rc;
  PrepareMixedArgs a{k, kr, batch * nk * d, v, static_cast<__half*>(vt16), scale, block_max,
                     batch, nk, dv, nk_pitch, v_kmajor ? 1 : 0, nullptr, nullptr, d, d, 0};
  const size_t v_blocks = v_kmajor ? batch * dv : batch * ((nk_pitch + 63) / 64) * ((dv + 63) / 64);
  const size_t most = std::max(batch * nk * d / 4 / 256 + 1, v_blocks);
  const size_t cap = static_cast<size_t>(kNumSMs) * 8;
  // Launched so that it may overlap the maxima kernel (see the wait in its V half).
  cudaLaunchAttribute overlap{};
  overlap.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  overlap.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(std::min(most, cap)), 2);
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cfg.attrs = &overlap;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, prepare_attention_mixed_kernel, a) != cudaSuccess)
    return fail(std::string("prepare_attention_operands_mixed: ") + cudaGetErrorString(cudaGetLastError()));
  count_launch();
  return 0;
}

int prepare_attention_operands_f16(const float* k, void* k16, float* k_tile_scale, const float* v,
                                   void* vt16, float* v_scale, float* block_max, size_t batch,
                                   size_t nk, size_t d, size_t dv, size_t d_pitch, size_t nk_pitch,
                                   bool v_kmajor, cudaStream_t s) {
  dim3 agrid(static_cast<unsigned>(batch), absmax_blocks_per_head(nk * dv));
  absmax_heads_kernel<<<agrid, 256, 0, s>>>(v, block_max, nk * dv);
  if (int rc = check_launch("absmax_heads")) return rc;
  const size_t kv_tiles = (nk + 127) / 128;
  PrepareMixedArgs a{k, nullptr, batch * nk * d, v, static_cast<__half*>(vt16), v_scale, block_max,
                     batch, nk, dv, nk_pitch, v_kmajor ? 1 : 0,
                     static_cast<__half*>(k16), k_tile_scale, d, d_pitch, kv_tiles};
  const size_t v_blocks = v_kmajor ? batch * dv : batch * ((nk_pitch + 63) / 64);
  const size_t cap = static_cast<size_t>(kNumSMs) * 8;
  // Launched so that it may overlap the maxima kernel (see the wait in the V half).
  cudaLaunchAttribute overlap{};
  overlap.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  overlap.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cfg.attrs = &overlap;
  cfg.numAttrs = 1;
  cudaError_t launched;
  if (batch * kv_tiles <= 512) {
    // Few tiles: one grid, both halves, K tiles held in registers.
    cfg.gridDim = dim3(static_cast<unsigned>(std::min(std::max(batch * kv_tiles, v_blocks), cap)), 2);
    launched = cudaLaunchKernelEx(&cfg, prepare_attention_f16_kernel<true>, a, 3);
  } else {
    // Many tiles: K with each tile held in registers (128 registers: in one grid with the V half
    // it would halve that half's occupancy; with two passes per tile instead it measured 1.8x the
    // bf16 conversion's time), running beside the maxima kernel, which it does not need but whose
    // completion it waits for before it ends; then V, which waits for the K grid and so for the
    // maxima.  The attention kernel that waits for the V grid thereby waits for all three.
    cfg.gridDim = dim3(static_cast<unsigned>(std::min(batch * kv_tiles, cap * 2)), 1);
    launched = cudaLaunchKernelEx(&cfg, prepare_attention_f16_kernel<true>, a, 1);
    if (launched == cudaSuccess) {
      count_launch();
      cfg.gridDim = dim3(static_cast<unsigned>(std::min(v_blocks, cap)), 1);
      launched = cudaLaunchKernelEx(&cfg, prepare_attention_f16_kernel<false>, a, 2);
    }
  }
  if (launched != cudaSuccess)
    return fail(std::string("prepare_attention_operands_f16: ") + cudaGetErrorString(cudaGetLastError()));
  count_launch();
  return 0;
}

int convert_bf16_rows(const float* in, void* out, size_t rows, size_t cols, size_t out_pitch,
                      cudaStream_t s) {
  if (rows == 0 || cols == 0) return 0;
  size_t blocks = (rows * (out_pitch / 4) + 255) / 256;
  if (blocks > static_cast<size_t>(kNumSMs) * 16) blocks = static_cast<size_t>(kNumSMs) * 16;
  convert_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
      in, static_cast<__nv_bfloat16*>(out), rows, cols, out_pitch);
  return check_launch("convert_bf16");
}

int convert_f16_rows_scaled(const float* in, void* out, float* scale, size_t rows, size_t cols,
                            size_t out_pitch, cudaStream_t s) {
  if (rows == 0 || cols == 0) return 0;
  size_t blocks = (rows + 7) / 8;
  if (blocks > static_cast<size_t>(kNumSMs) * 64) blocks = static_cast<size_t>(kNumSMs) * 64;
  convert_f16_rows_scaled_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
      in, static_cast<__half*>(out), scale, rows, cols, out_pitch);
  return check_launch("convert_f16_rows_scaled");
}

int prepare_attention_operands(const float* q, float* qr, size_t q_elems, const float* k,
                               float* kr, size_t k_elems, const float* v, float* vt, size_t batch,
                               size_t nk, size_t dv, size_t pitch, cudaStream_t s) {
  PrepareArgs a{q, qr, q_elems, k, kr, k_elems, v, vt, batch, nk, dv, pitch};
  const size_t most = std::max(std::max(q_elems, k_elems) / 4 / 256 + 1,
                               batch * ((nk + 63) / 64) * ((dv + 63) / 64));
  const size_t cap = static_cast<size_t>(kNumSMs) * 8;
  dim3 grid(static_cast<unsigned>(std::min(most, cap)), 3);
  prepare_attention_kernel<<<grid, 256, 0, s>>>(a);
  return check_launch("prepare_attention_operands");
}

int round_tf32_rows(const float* in0, float* out0, size_t rows0, size_t cols0, size_t in_pitch0,
                    size_t out_pitch0, const float* in1, float* out1, size_t rows1, size_t cols1,
                    size_t in_pitch1, size_t out_pitch1, cudaStream_t s) {
  RoundJob j0{in0, out0, rows0, cols0, in_pitch0, out_pitch0};
  RoundJob j1{in1, out1, rows1, cols1, in_pitch1, out_pitch1};
  const size_t n = std::max(rows0 * cols0, in1 ? rows1 * cols1 : 0);
  if (n == 0) return 0;
  size_t blocks = (n / 4 + 255) / 256 + 1;
  if (blocks > static_cast<size_t>(kNumSMs) * 16) blocks = static_cast<size_t>(kNumSMs) * 16;
  dim3 grid(static_cast<unsigned>(blocks), in1 ? 2 : 1);
  round_rows_kernel<<<grid, 256, 0, s>>>(j0, j1);
  return check_launch("round_tf32");
}

int contract_simt(const float* a, const float* b, float* c, size_t batch, size_t m, size_t n,
                  size_t k, bool a_kmajor, bool b_kmajor, cudaStream_t s, size_t splits) {
  if (batch == 0 || m == 0 || n == 0) return 0;
  if (splits < 1) splits = 1;
  if (batch * splits > 65535) return fail("ib_contract: more than 65535 batch entries");
  // Whole k-tiles per split, so that every split but the last is full.
  const size_t k_len = ((k + splits - 1) / splits + kTileK - 1) / kTileK * kTileK;
  dim3 grid(static_cast<unsigned>((n + kTile - 1) / kTile),
            static_cast<unsigned>((m + kTile - 1) / kTile), static_cast<unsigned>(batch * splits));
  if (grid.y > 65535) return fail("ib_contract: row count too large for the fp32 arm");
  if (a_kmajor && b_kmajor)
    contract_simt_kernel<true, true><<<grid, 256, 0, s>>>(a, b, c, m, n, k, splits, k_len);
  else if (a_kmajor && !b_kmajor)
    contract_simt_kernel<true, false><<<grid, 256, 0, s>>>(a, b, c, m, n, k, splits, k_len);
  else if (!a_kmajor && b_kmajor)
    contract_simt_kernel<false, true><<<grid, 256, 0, s>>>(a, b, c, m, n, k, splits, k_len);
  else
    contract_simt_kernel<false, false><<<grid, 256, 0, s>>>(a, b, c, m, n, k, splits, k_len);
  return check_launch("ib_contract (fp32)");
}

int transpose_batched(const float* in, float* out, size_t batch, size_t rows, size_t cols,
                      size_t out_pitch, bool round, cudaStream_t s) {
  if (batch == 0 || rows == 0 || cols == 0) return 0;
  if (batch > 65535 || (rows + 63) / 64 > 65535) return fail("transpose: shape too large");
  dim3 grid(static_cast<unsigned>((cols + 63) / 64), static_cast<unsigned>((rows + 63) / 64),
            static_cast<unsigned>(batch));
  // 16-byte accesses need every row of either side, in every batch entry, to start on 16 bytes.
  const bool vec = cols % 4 == 0 && out_pitch % 4 == 0 && (rows * cols) % 4 == 0 &&
                   (reinterpret_cast<uintptr_t>(in) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
  if (round)
    transpose_kernel<true><<<grid, 256, 0, s>>>(in, out, rows, cols, out_pitch, vec);
  else
    transpose_kernel<false><<<grid, 256, 0, s>>>(in, out, rows, cols, out_pitch, vec);
  return check_launch("transpose");
}

}  // namespace ib
