// Row reductions `+ * > < && || ^^` over the last axis, and a general strided fold.
//
// Identities and accumulate form follow the reference
// (compiler/src/lower/exec_plan_to_module.rs:592-603, 354-367): the fold starts
// from the op's identity and applies dst = op(dst, x).  The reference folds in
// ascending column order on one thread; here a row is folded as a tree across
// lanes, which is exact for max/min and differs from the sequential float sum
// only by rounding.  Algorithmic traffic: rows*cols*4 + rows*4 bytes.  Eight 16-byte loads in
// flight per thread and one CTA per row (no cap on the grid) measured 5.6-5.85 TB/s on B200 against
// 5.2 for two loads per thread on a grid capped at 16 CTAs per SM.
#include "common.cuh"

namespace ib {
namespace {

#ifndef IB_RED_UNROLL
#define IB_RED_UNROLL 8
#endif
#ifndef IB_RED_CAP
#define IB_RED_CAP 65536
#endif
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = IB_RED_UNROLL;   // 16-byte loads in flight per thread in the one-row-per-CTA kernel

// One warp per row: rows of up to a few thousand columns.
template <int OP>
__global__ void __launch_bounds__(kThreads)
reduce_rows_warp(const float* __restrict__ x, float* __restrict__ y, size_t rows, size_t cols,
                 bool vec) {
  const int lane = threadIdx.x & 31;
  const size_t warps_total = static_cast<size_t>(gridDim.x) * kWarps;
  for (size_t r = static_cast<size_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5); r < rows;
       r += warps_total) {
    const float* row = x + r * cols;
    float acc = reduce_identity(OP);
    if (vec) {
      const float4* row4 = reinterpret_cast<const float4*>(row);
      const size_t nvec = cols / 4;
      constexpr int kWarpUnroll = 4;          // 16-byte loads in flight per lane
      size_t i = lane;
      for (; i + (kWarpUnroll - 1) * 32 < nvec; i += kWarpUnroll * 32) {
        float4 v[kWarpUnroll];
#pragma unroll
        for (int u = 0; u < kWarpUnroll; ++u) v[u] = __ldcs(row4 + i + u * 32);
#pragma unroll
        for (int u = 0; u < kWarpUnroll; ++u)
          acc = fold<OP>(acc, fold<OP>(fold<OP>(v[u].x, v[u].y), fold<OP>(v[u].z, v[u].w)));
      }
      for (; i < nvec; i += 32) {
        float4 v = __ldcs(row4 + i);
        acc = fold<OP>(acc, fold<OP>(fold<OP>(v.x, v.y), fold<OP>(v.z, v.w)));
      }
    } else {
      for (size_t i = lane; i < cols; i += 32) acc = fold<OP>(acc, row[i]);
    }
    acc = warp_fold<OP>(acc);
    if (lane == 0) y[r] = acc;
  }
}

// One CTA per row: long rows.
template <int OP>
__global__ void __launch_bounds__(kThreads)
reduce_rows_block(const float* __restrict__ x, float* __restrict__ y, size_t rows, size_t cols,
                  bool vec) {
  __shared__ float partial[kWarps];
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* row = x + r * cols;
    float accs[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) accs[u] = reduce_identity(OP);
    if (vec) {
      const float4* row4 = reinterpret_cast<const float4*>(row);
      const size_t nvec = cols / 4;
      size_t i = threadIdx.x;
      for (; i + (kUnroll - 1) * kThreads < nvec; i += kUnroll * kThreads) {
        float4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = __ldcs(row4 + i + u * kThreads);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          accs[u] = fold<OP>(accs[u], fold<OP>(fold<OP>(v[u].x, v[u].y), fold<OP>(v[u].z, v[u].w)));
      }
      for (; i < nvec; i += kThreads) {
        const float4 v = __ldcs(row4 + i);
        accs[0] = fold<OP>(accs[0], fold<OP>(fold<OP>(v.x, v.y), fold<OP>(v.z, v.w)));
      }
    } else {
      for (size_t i = threadIdx.x; i < cols; i += kThreads) accs[0] = fold<OP>(accs[0], row[i]);
    }
    float acc0 = accs[0];
#pragma unroll
    for (int u = 1; u < kUnroll; ++u) acc0 = fold<OP>(acc0, accs[u]);
    float acc = warp_fold<OP>(acc0);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
      float v = threadIdx.x < kWarps ? partial[threadIdx.x] : reduce_identity(OP);
      v = warp_fold<OP>(v);
      if (threadIdx.x == 0) y[r] = v;
    }
    __syncthreads();
  }
}

struct FoldArgs {
  int kept_rank, red_rank;
  size_t kept_extent[IB_MAX_RANK];
  ptrdiff_t kept_stride[IB_MAX_RANK];
  size_t red_extent[IB_MAX_RANK];
  ptrdiff_t red_stride[IB_MAX_RANK];
};

// One warp per result element, lanes striding over the flattened reduced space.
template <int OP>
__global__ void __launch_bounds__(kThreads)
reduce_strided(const float* __restrict__ x, float* __restrict__ y, size_t n_out, size_t n_red,
               FoldArgs args) {
  const int lane = threadIdx.x & 31;
  const size_t warps_total = static_cast<size_t>(gridDim.x) * kWarps;
  for (size_t o = static_cast<size_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5); o < n_out;
       o += warps_total) {
    size_t rest = o;
    ptrdiff_t base = 0;
    for (int d = args.kept_rank - 1; d >= 0; --d) {
      size_t q = rest / args.kept_extent[d];
      base += static_cast<ptrdiff_t>(rest - q * args.kept_extent[d]) * args.kept_stride[d];
      rest = q;
    }
    float acc = reduce_identity(OP);
    for (size_t i = lane; i < n_red; i += 32) {
      size_t left = i;
      ptrdiff_t off = base;
      for (int d = args.red_rank - 1; d >= 0; --d) {
        size_t q = left / args.red_extent[d];
        off += static_cast<ptrdiff_t>(left - q * args.red_extent[d]) * args.red_stride[d];
        left = q;
      }
      acc = fold<OP>(acc, x[off]);
    }
    acc = warp_fold<OP>(acc);
    if (lane == 0) y[o] = acc;
  }
}

template <int OP>
int launch_rows(const float* x, float* y, size_t rows, size_t cols, cudaStream_t s) {
  const bool vec = cols % 4 == 0 && aligned16(x);
  if (cols <= 2048) {
    size_t blocks = (rows + kWarps - 1) / kWarps;
    size_t cap = static_cast<size_t>(kNumSMs) * IB_RED_CAP;
    reduce_rows_warp<OP><<<static_cast<int>(blocks < cap ? blocks : cap), kThreads, 0, s>>>(
        x, y, rows, cols, vec);
  } else {
    size_t cap = static_cast<size_t>(kNumSMs) * IB_RED_CAP;
    reduce_rows_block<OP><<<static_cast<int>(rows < cap ? rows : cap), kThreads, 0, s>>>(
        x, y, rows, cols, vec);
  }
  return check_launch("ib_reduce_rows");
}

template <int OP>
int launch_strided(const float* x, float* y, size_t n_out, size_t n_red, const FoldArgs& args,
                   cudaStream_t s) {
  size_t blocks = (n_out + kWarps - 1) / kWarps;
  size_t cap = static_cast<size_t>(kNumSMs) * IB_RED_CAP;
  reduce_strided<OP><<<static_cast<int>(blocks < cap ? blocks : cap), kThreads, 0, s>>>(
      x, y, n_out, n_red, args);
  return check_launch("ib_reduce_strided");
}

}  // namespace
}  // namespace ib

#define IB_DISPATCH_FOLD(op, CALL)                                             \
  switch (op) {                                                                \
    case IB_OP_ADD: return CALL(IB_OP_ADD);                                    \
    case IB_OP_MUL: return CALL(IB_OP_MUL);                                    \
    case IB_OP_MAX: return CALL(IB_OP_MAX);                                    \
    case IB_OP_MIN: return CALL(IB_OP_MIN);                                    \
    case IB_OP_AND: return CALL(IB_OP_AND);                                    \
    case IB_OP_OR: return CALL(IB_OP_OR);                                      \
    case IB_OP_XOR: return CALL(IB_OP_XOR);                                    \
    default: return ib::fail("operator is not reducible (only + * > < && || ^^ fold)"); \
  }

extern "C" int ib_reduce_rows(int op, const float* x, float* y, size_t rows, size_t cols,
                              void* stream) {
  if (rows == 0) return 0;
  if (!y || (!x && cols != 0)) return ib::fail("ib_reduce_rows: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CALL(OP) ib::launch_rows<OP>(x, y, rows, cols, s)
  IB_DISPATCH_FOLD(op, CALL)
#undef CALL
}

extern "C" int ib_reduce_strided(int op, const float* x, float* y, int kept_rank,
                                 const size_t* kept_extent, const ptrdiff_t* kept_stride,
                                 int red_rank, const size_t* red_extent,
                                 const ptrdiff_t* red_stride, void* stream) {
  if (kept_rank < 0 || kept_rank > IB_MAX_RANK || red_rank < 0 || red_rank > IB_MAX_RANK)
    return ib::fail("ib_reduce_strided: rank out of range");
  if (!x || !y) return ib::fail("ib_reduce_strided: null pointer");
  ib::FoldArgs args{};
  args.kept_rank = kept_rank;
  args.red_rank = red_rank;
  size_t n_out = 1, n_red = 1;
  for (int d = 0; d < kept_rank; ++d) {
    args.kept_extent[d] = kept_extent[d];
    args.kept_stride[d] = kept_stride[d];
    n_out *= kept_extent[d];
  }
  for (int d = 0; d < red_rank; ++d) {
    args.red_extent[d] = red_extent[d];
    args.red_stride[d] = red_stride[d];
    n_red *= red_extent[d];
  }
  if (n_out == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CALL(OP) ib::launch_strided<OP>(x, y, n_out, n_red, args, s)
  IB_DISPATCH_FOLD(op, CALL)
#undef CALL
}
