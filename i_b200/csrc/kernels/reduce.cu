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
// WEIGHT: what is folded is x itself (kPlain), x times a second array of the same shape
// (kTimesRows: row-wise dot products) or x times one vector of `cols` values (kTimesVector: matrix
// times vector).  The product is rounded before it is added, as the reference's `tmp = a * b;
// c = c + tmp` is (ilang-python/annotated-flashattn.c:67-85).
enum Weight { kPlain, kTimesRows, kTimesVector };

template <int WEIGHT>
__device__ __forceinline__ float4 weighted(float4 v, const float4* w_row4, const float4* w_vec4, size_t i) {
  if (WEIGHT == kPlain) return v;
  const float4 w = WEIGHT == kTimesRows ? __ldcs(w_row4 + i) : __ldg(w_vec4 + i);
  return make_float4(__fmul_rn(v.x, w.x), __fmul_rn(v.y, w.y), __fmul_rn(v.z, w.z), __fmul_rn(v.w, w.w));
}

template <int OP, int WEIGHT = kPlain>
__global__ void __launch_bounds__(kThreads)
reduce_rows_warp(const float* __restrict__ x, float* __restrict__ y, size_t rows, size_t cols,
                 bool vec, const float* __restrict__ w = nullptr) {
  const int lane = threadIdx.x & 31;
  const size_t warps_total = static_cast<size_t>(gridDim.x) * kWarps;
  if (vec && cols <= 128) {
    // Rows of one 16-byte load per lane: a warp takes four rows at a time, so that four loads
    // per lane are in flight instead of one (2^20 x 100: 190 us with one row at a time).
    constexpr int kRowsAtOnce = 4;
    const size_t nvec = cols / 4;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    for (size_t r0 = (static_cast<size_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5)) * kRowsAtOnce; r0 < rows;
         r0 += warps_total * kRowsAtOnce) {
      float acc[kRowsAtOnce];
#pragma unroll
      for (int u = 0; u < kRowsAtOnce; ++u) {
        acc[u] = reduce_identity(OP);
        const size_t r = r0 + u;
        if (r < rows && static_cast<size_t>(lane) < nvec) {
          const float4* row4 = reinterpret_cast<const float4*>(x + r * cols);
          const float4 v = weighted<WEIGHT>(__ldcs(row4 + lane), w4 + (WEIGHT == kTimesRows ? r * nvec : 0),
                                            w4, lane);
          acc[u] = fold<OP>(fold<OP>(v.x, v.y), fold<OP>(v.z, v.w));
        }
      }
#pragma unroll
      for (int u = 0; u < kRowsAtOnce; ++u) {
        const float total = warp_fold<OP>(acc[u]);
        if (lane == 0 && r0 + u < rows) y[r0 + u] = total;
      }
    }
    return;
  }
  for (size_t r = static_cast<size_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5); r < rows;
       r += warps_total) {
    const float* row = x + r * cols;
    const float* wrow = WEIGHT == kTimesRows ? w + r * cols : w;
    float acc = reduce_identity(OP);
    if (vec) {
      const float4* row4 = reinterpret_cast<const float4*>(row);
      const float4* w4 = reinterpret_cast<const float4*>(wrow);
      const size_t nvec = cols / 4;
      constexpr int kWarpUnroll = 4;          // 16-byte loads in flight per lane
      size_t i = lane;
      for (; i + (kWarpUnroll - 1) * 32 < nvec; i += kWarpUnroll * 32) {
        float4 v[kWarpUnroll];
#pragma unroll
        for (int u = 0; u < kWarpUnroll; ++u)
          v[u] = weighted<WEIGHT>(__ldcs(row4 + i + u * 32), w4, w4, i + u * 32);
#pragma unroll
        for (int u = 0; u < kWarpUnroll; ++u)
          acc = fold<OP>(acc, fold<OP>(fold<OP>(v[u].x, v[u].y), fold<OP>(v[u].z, v[u].w)));
      }
      for (; i < nvec; i += 32) {
        float4 v = weighted<WEIGHT>(__ldcs(row4 + i), w4, w4, i);
        acc = fold<OP>(acc, fold<OP>(fold<OP>(v.x, v.y), fold<OP>(v.z, v.w)));
      }
    } else {
      for (size_t i = lane; i < cols; i += 32)
        acc = fold<OP>(acc, WEIGHT == kPlain ? row[i] : __fmul_rn(row[i], wrow[i]));
    }
    acc = warp_fold<OP>(acc);
    if (lane == 0) y[r] = acc;
  }
}

// One CTA per row: long rows.
// A row may be cut into `segs` segments of `seg_len` columns (a multiple of four; the last one
// shorter), each folded by a CTA of its own into y[row * segs + segment]: few rows of millions of
// columns (a sum over a whole array) would otherwise keep one CTA each busy and the rest idle.
template <int OP, int WEIGHT = kPlain>
__global__ void __launch_bounds__(kThreads)
reduce_rows_block(const float* __restrict__ x, float* __restrict__ y, size_t rows, size_t cols,
                  bool vec, const float* __restrict__ w = nullptr, size_t segs = 1, size_t seg_len = 0) {
  __shared__ float partial[kWarps];
  for (size_t r = blockIdx.x; r < rows * segs; r += gridDim.x) {
    const size_t whole = r / segs, at = (r - whole * segs) * seg_len;
    const size_t len = segs == 1 ? cols : (cols - at < seg_len ? cols - at : seg_len);
    const float* row = x + whole * cols + at;
    const float* wrow = WEIGHT == kTimesRows ? w + whole * cols + at : w + at;
    float accs[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) accs[u] = reduce_identity(OP);
    if (vec) {
      const float4* row4 = reinterpret_cast<const float4*>(row);
      const float4* w4 = reinterpret_cast<const float4*>(wrow);
      const size_t nvec = len / 4;
      size_t i = threadIdx.x;
      for (; i + (kUnroll - 1) * kThreads < nvec; i += kUnroll * kThreads) {
        float4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          v[u] = weighted<WEIGHT>(__ldcs(row4 + i + u * kThreads), w4, w4, i + u * kThreads);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          accs[u] = fold<OP>(accs[u], fold<OP>(fold<OP>(v[u].x, v[u].y), fold<OP>(v[u].z, v[u].w)));
      }
      for (; i < nvec; i += kThreads) {
        const float4 v = weighted<WEIGHT>(__ldcs(row4 + i), w4, w4, i);
        accs[0] = fold<OP>(accs[0], fold<OP>(fold<OP>(v.x, v.y), fold<OP>(v.z, v.w)));
      }
    } else {
      for (size_t i = threadIdx.x; i < len; i += kThreads)
        accs[0] = fold<OP>(accs[0], WEIGHT == kPlain ? row[i] : __fmul_rn(row[i], wrow[i]));
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

// Segments per row for few, very long rows (1 = the row stays whole): enough CTAs to fill the
// machine, at least 8192 columns each, a multiple of four columns long.
struct RowSplit {
  size_t segs = 1, seg_len = 0;
};
RowSplit split_long_rows(size_t rows, size_t cols) {
  RowSplit sp;
  const size_t want = static_cast<size_t>(kNumSMs) * 8;
  if (rows == 0 || rows >= static_cast<size_t>(kNumSMs) * 2 || cols < 4 * 8192) return sp;
  size_t segs = (want + rows - 1) / rows;
  if (segs > cols / 8192) segs = cols / 8192;
  if (segs < 2) return sp;
  sp.seg_len = ((cols + segs - 1) / segs + 3) / 4 * 4;
  sp.segs = (cols + sp.seg_len - 1) / sp.seg_len;
  return sp;
}

template <int OP, int WEIGHT>
int launch_rows_split(const float* x, const float* w, float* y, size_t rows, size_t cols, float* partials,
                      cudaStream_t s) {
  const RowSplit sp = split_long_rows(rows, cols);
  const bool vec = cols % 4 == 0 && aligned16(x) && (WEIGHT == kPlain || aligned16(w));
  const size_t cap = static_cast<size_t>(kNumSMs) * IB_RED_CAP;
  const size_t ctas = rows * sp.segs;
  reduce_rows_block<OP, WEIGHT><<<static_cast<int>(ctas < cap ? ctas : cap), kThreads, 0, s>>>(
      x, partials, rows, cols, vec, w, sp.segs, sp.seg_len);
  if (int rc = check_launch("ib_reduce_rows (segments)")) return rc;
  const size_t blocks = (rows + kWarps - 1) / kWarps;
  reduce_rows_warp<OP><<<static_cast<int>(blocks < cap ? blocks : cap), kThreads, 0, s>>>(
      partials, y, rows, sp.segs, sp.segs % 4 == 0 && aligned16(partials));
  return check_launch("ib_reduce_rows (partials)");
}

template <int OP>
int launch_rows(const float* x, float* y, size_t rows, size_t cols, cudaStream_t s,
                float* partials = nullptr) {
  if (partials && split_long_rows(rows, cols).segs > 1)
    return launch_rows_split<OP, kPlain>(x, nullptr, y, rows, cols, partials, s);
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

template <int WEIGHT>
int launch_dot_rows(const float* x, const float* w, float* y, size_t rows, size_t cols, cudaStream_t s,
                    float* partials) {
  if (partials && split_long_rows(rows, cols).segs > 1)
    return launch_rows_split<IB_OP_ADD, WEIGHT>(x, w, y, rows, cols, partials, s);
  const bool vec = cols % 4 == 0 && aligned16(x) && aligned16(w);
  const size_t cap = static_cast<size_t>(kNumSMs) * IB_RED_CAP;
  if (cols <= 2048) {
    const size_t blocks = (rows + kWarps - 1) / kWarps;
    reduce_rows_warp<IB_OP_ADD, WEIGHT><<<static_cast<int>(blocks < cap ? blocks : cap), kThreads, 0, s>>>(
        x, y, rows, cols, vec, w);
  } else {
    reduce_rows_block<IB_OP_ADD, WEIGHT><<<static_cast<int>(rows < cap ? rows : cap), kThreads, 0, s>>>(
        x, y, rows, cols, vec, w);
  }
  return check_launch("ib_contract (rows)");
}

// ---- folds of the leading axis: y[c] = fold over r of x[r][c] (`+ij~j`, `+bij~ij`) ------------
//
// A thread owns four neighbouring columns and walks down a slab of rows, eight 16-byte loads in
// flight; the threads of a CTA that one row does not fill take further rows (narrow arrays: a row
// of 64 columns is 16 threads wide, so a CTA walks 16 rows at a time) and meet in shared memory.
// The rows are cut into slabs so that the grid fills the machine; with more than one slab the
// kernel writes one partial row per slab and runs once more over those.  The order of the fold is
// fixed by the shape alone, so results repeat from run to run (no atomics).  ROW_WEIGHT:
// x[r][c] * w[r] is folded instead of x[r][c] (vector times matrix, the product rounded before it
// is added).  Algorithmic traffic: rows*cols*4 + cols*4 bytes.
constexpr int kColsUnroll = 8;

template <int OP, bool ROW_WEIGHT, bool VEC>
__global__ void __launch_bounds__(kThreads)
fold_leading_axis(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                  size_t rows, size_t cols, size_t rows_per_slab, int lanes_log2) {
  constexpr int kWidth = VEC ? 4 : 1;
  __shared__ float meet[kThreads][kWidth];
  // blockIdx.z: one of several arrays of the same shape, one behind the other (`+bij~bj`).
  x += static_cast<size_t>(blockIdx.z) * rows * cols;
  y += static_cast<size_t>(blockIdx.z) * gridDim.y * cols;
  // lanes = 2^lanes_log2 threads side by side cover a row's columns in this CTA; kThreads / lanes
  // rows are in flight at a time.
  const int lanes = 1 << lanes_log2;
  const int tx = threadIdx.x & (lanes - 1), ty = threadIdx.x >> lanes_log2;
  const size_t phases = kThreads >> lanes_log2;
  const size_t c = (static_cast<size_t>(blockIdx.x) * lanes + tx) * kWidth;
  const bool live = c < cols;
  const size_t r_lo = static_cast<size_t>(blockIdx.y) * rows_per_slab;
  const size_t r_hi = r_lo + rows_per_slab < rows ? r_lo + rows_per_slab : rows;
  float acc[kWidth];
#pragma unroll
  for (int e = 0; e < kWidth; ++e) acc[e] = reduce_identity(OP);
  auto take = [&](size_t r, float (&v)[kWidth]) {
    if (VEC) {
      const float4 q = __ldcs(reinterpret_cast<const float4*>(x + r * cols + c));
      v[0] = q.x;
      if (kWidth == 4) { v[1] = q.y; v[2] = q.z; v[3] = q.w; }
    } else {
      v[0] = x[r * cols + c];
    }
    if (ROW_WEIGHT) {
      const float s = __ldg(w + r);
#pragma unroll
      for (int e = 0; e < kWidth; ++e) v[e] = __fmul_rn(v[e], s);
    }
  };
  if (live) {
    size_t r = r_lo + ty;
    for (; r + (kColsUnroll - 1) * phases < r_hi; r += kColsUnroll * phases) {
      float v[kColsUnroll][kWidth];
#pragma unroll
      for (int u = 0; u < kColsUnroll; ++u) take(r + u * phases, v[u]);
#pragma unroll
      for (int u = 0; u < kColsUnroll; ++u)
#pragma unroll
        for (int e = 0; e < kWidth; ++e) acc[e] = fold<OP>(acc[e], v[u][e]);
    }
    for (; r < r_hi; r += phases) {
      float v[kWidth];
      take(r, v);
#pragma unroll
      for (int e = 0; e < kWidth; ++e) acc[e] = fold<OP>(acc[e], v[e]);
    }
  }
  if (phases > 1) {
#pragma unroll
    for (int e = 0; e < kWidth; ++e) meet[threadIdx.x][e] = acc[e];
    __syncthreads();
    if (ty != 0) return;
    for (size_t p = 1; p < phases; ++p)
#pragma unroll
      for (int e = 0; e < kWidth; ++e) acc[e] = fold<OP>(acc[e], meet[p * lanes + tx][e]);
  }
  if (!live) return;
  float* dst = y + static_cast<size_t>(blockIdx.y) * cols + c;
  if (VEC) {
    *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[kWidth > 1 ? 1 : 0], acc[kWidth > 2 ? 2 : 0],
                                                  acc[kWidth > 3 ? 3 : 0]);
  } else {
    dst[0] = acc[0];
  }
}

// Threads of a CTA side by side on one row, as a power of two: as many as the row has column
// groups (of four columns when `vec`), at most the whole CTA.
int leading_axis_lanes_log2(size_t cols, bool vec) {
  const size_t groups = vec ? cols / 4 : cols;
  int l = 0;
  while ((1u << l) < kThreads && (static_cast<size_t>(1) << l) < groups) ++l;
  return l;
}

// Slabs of rows for a fold of `rows` x `cols`: enough CTAs to fill the machine several times
// over, every thread with at least 16 rows.  (Sized for the four-column form; the one-column
// form of the same shape has more CTAs per slab and fills the machine sooner.)
size_t leading_axis_slabs(size_t rows, size_t cols, size_t batch = 1) {
  const int l = leading_axis_lanes_log2(cols, cols % 4 == 0);
  const size_t groups = cols % 4 == 0 ? cols / 4 : cols;
  const size_t col_blocks = ((groups + (1u << l) - 1) >> l) * (batch ? batch : 1);
  const size_t phases = kThreads >> l;
  size_t slabs = (static_cast<size_t>(kNumSMs) * 8 + col_blocks - 1) / col_blocks;
  if (slabs > rows / (16 * phases)) slabs = rows / (16 * phases);
  if (slabs > 65535) slabs = 65535;
  return slabs < 1 ? 1 : slabs;
}

template <int OP, bool ROW_WEIGHT>
int launch_leading_axis_once(const float* x, const float* w, float* y, size_t rows, size_t cols,
                             size_t rows_per_slab, size_t slabs, cudaStream_t s, size_t batch = 1) {
  const bool vec = cols % 4 == 0 && aligned16(x) && aligned16(y);
  int l = leading_axis_lanes_log2(cols, vec);
  const size_t groups = vec ? cols / 4 : cols;
  // One slab (the fold of the slabs' results, or too few rows to cut): narrower CTAs, down to
  // eight threads side by side (a 128-byte line per row), until the grid covers the machine;
  // the threads this frees walk further rows (147 partial rows of 8192 columns on eight CTAs of
  // full width took 32 us, three quarters of the fold that produced them).
  if (slabs == 1)
    while (l > 3 && ((groups + (1u << l) - 1) >> l) * batch < 2 * static_cast<size_t>(kNumSMs) &&
           rows_per_slab >= (static_cast<size_t>(kThreads) >> (l - 1)))
      --l;
  dim3 grid(static_cast<unsigned>((groups + (1u << l) - 1) >> l), static_cast<unsigned>(slabs),
            static_cast<unsigned>(batch));
  if (vec)
    fold_leading_axis<OP, ROW_WEIGHT, true><<<grid, kThreads, 0, s>>>(x, w, y, rows, cols, rows_per_slab, l);
  else
    fold_leading_axis<OP, ROW_WEIGHT, false><<<grid, kThreads, 0, s>>>(x, w, y, rows, cols, rows_per_slab, l);
  return check_launch("ib_reduce_leading");
}

template <int OP, bool ROW_WEIGHT>
int launch_leading_axis(const float* x, const float* w, float* y, size_t rows, size_t cols,
                        float* partials, cudaStream_t s, size_t batch = 1) {
  if (batch > 65535) return fail("ib_reduce_leading: more than 65535 arrays");
  const size_t slabs = partials ? leading_axis_slabs(rows, cols, batch) : 1;
  const size_t rows_per_slab = (rows + slabs - 1) / slabs;
  const size_t used = rows_per_slab ? (rows + rows_per_slab - 1) / rows_per_slab : 1;   // slabs that hold rows
  if (used <= 1)
    return launch_leading_axis_once<OP, ROW_WEIGHT>(x, w, y, rows, cols, rows ? rows : 1, 1, s, batch);
  if (int rc = launch_leading_axis_once<OP, ROW_WEIGHT>(x, w, partials, rows, cols, rows_per_slab, used, s,
                                                        batch))
    return rc;
  // The partial rows, one per slab, folded the same way as one slab.
  return launch_leading_axis_once<OP, false>(partials, nullptr, y, used, cols, used, 1, s, batch);
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

size_t dot_leading_axis_floats(size_t rows, size_t cols) {
  const size_t slabs = leading_axis_slabs(rows, cols);
  return slabs > 1 ? slabs * cols : 0;
}

int dot_leading_axis(const float* x, const float* w, float* y, size_t rows, size_t cols,
                     float* partials, cudaStream_t s) {
  if (cols == 0) return 0;
  return launch_leading_axis<IB_OP_ADD, true>(x, w, y, rows, cols, partials, s);
}

int sum_partials(const float* x, float* y, size_t batch, size_t rows, size_t cols, cudaStream_t s) {
  if (batch == 0 || cols == 0) return 0;
  return launch_leading_axis<IB_OP_ADD, false>(x, nullptr, y, rows, cols, nullptr, s, batch);
}

size_t long_rows_floats(size_t rows, size_t cols) {
  const RowSplit sp = split_long_rows(rows, cols);
  return sp.segs > 1 ? rows * sp.segs : 0;
}

int dot_rows(const float* x, const float* w, bool w_is_vector, float* y, size_t rows, size_t cols,
             cudaStream_t s, float* partials) {
  if (rows == 0) return 0;
  return w_is_vector ? launch_dot_rows<kTimesVector>(x, w, y, rows, cols, s, partials)
                     : launch_dot_rows<kTimesRows>(x, w, y, rows, cols, s, partials);
}

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

extern "C" size_t ib_reduce_rows_workspace_bytes(size_t rows, size_t cols) {
  return ib::long_rows_floats(rows, cols) * sizeof(float);
}

extern "C" int ib_reduce_rows_split(int op, const float* x, float* y, size_t rows, size_t cols,
                                    void* workspace, size_t workspace_bytes, void* stream) {
  if (rows == 0) return 0;
  if (!y || (!x && cols != 0)) return ib::fail("ib_reduce_rows: null pointer");
  const size_t need = ib_reduce_rows_workspace_bytes(rows, cols);
  float* partials = need && workspace && workspace_bytes >= need ? static_cast<float*>(workspace) : nullptr;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CALL(OP) ib::launch_rows<OP>(x, y, rows, cols, s, partials)
  IB_DISPATCH_FOLD(op, CALL)
#undef CALL
}

extern "C" size_t ib_reduce_leading_workspace_bytes(size_t batch, size_t rows, size_t cols) {
  if (batch == 0 || cols == 0) return 0;
  if (rows > SIZE_MAX / sizeof(float) / cols / batch) return SIZE_MAX;
  const size_t slabs = ib::leading_axis_slabs(rows, cols, batch);
  return slabs > 1 ? batch * slabs * cols * sizeof(float) : 0;
}

extern "C" int ib_reduce_leading(int op, const float* x, float* y, size_t batch, size_t rows,
                                 size_t cols, void* workspace, size_t workspace_bytes, void* stream) {
  if (cols == 0 || batch == 0) return 0;
  if (!y || (!x && rows != 0)) return ib::fail("ib_reduce_leading: null pointer");
  // Without (enough) workspace the rows are folded as one slab: correct, slower on tall inputs.
  float* partials = workspace_bytes >= ib_reduce_leading_workspace_bytes(batch, rows, cols) && workspace_bytes > 0
                        ? static_cast<float*>(workspace)
                        : nullptr;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CALL(OP) ib::launch_leading_axis<OP, false>(x, nullptr, y, rows, cols, partials, s, batch)
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
