// Pointwise maps: memory-bound, 128-bit vectorised, eight 16-byte loads in flight per thread and
// one block per 32 KB of input (measured on B200 at 8192 x 8192: 6.0-6.1 TB/s against 5.5-5.8 for four
// loads per thread on a grid capped at 16 blocks per SM; a plain device copy by torch runs at 6.07).
//
// Scalar semantics follow the reference's lowering
// (compiler/src/lower/exec_plan_to_module.rs:605-640 for unary defaults,
// compiler/src/backends/c/expr.rs:127-148 for the binary spelling).
// Algorithmic traffic: (operands + 1) * elements * 4 bytes, a broadcast operand
// counted at its own size.
#include "common.cuh"

namespace ib {
namespace {

constexpr int kThreads = 256;
#ifndef IB_MAP_VEC
#define IB_MAP_VEC 8
#endif
#ifndef IB_MAP_CAP
#define IB_MAP_CAP 65536
#endif
constexpr int kVecPerThread = IB_MAP_VEC;  // float4 loads in flight per thread

inline int grid_for(size_t work_items, size_t per_block) {
  size_t blocks = (work_items + per_block - 1) / per_block;
  size_t cap = static_cast<size_t>(kNumSMs) * IB_MAP_CAP;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  return static_cast<int>(blocks);
}

template <int OP>
__global__ void __launch_bounds__(kThreads)
map_unary_vec(const float4* __restrict__ x, float4* __restrict__ y, size_t nvec) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads * kVecPerThread;
  for (size_t base = (static_cast<size_t>(blockIdx.x) * kThreads) * kVecPerThread + threadIdx.x;
       base < nvec; base += stride) {
    float4 v[kVecPerThread];
#pragma unroll
    for (int u = 0; u < kVecPerThread; ++u) {
      size_t i = base + static_cast<size_t>(u) * kThreads;
      if (i < nvec) v[u] = __ldcs(x + i);
    }
#pragma unroll
    for (int u = 0; u < kVecPerThread; ++u) {
      size_t i = base + static_cast<size_t>(u) * kThreads;
      if (i < nvec) {
        float4 r;
        r.x = apply_unary(OP, v[u].x);
        r.y = apply_unary(OP, v[u].y);
        r.z = apply_unary(OP, v[u].z);
        r.w = apply_unary(OP, v[u].w);
        __stcs(y + i, r);
      }
    }
  }
}

template <int OP>
__global__ void __launch_bounds__(kThreads)
map_unary_scalar(const float* __restrict__ x, float* __restrict__ y, size_t begin, size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = begin + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
       i += stride)
    y[i] = apply_unary(OP, x[i]);
}

// Element e of a rows x cols result reads a[e] or a[r] or a[c] depending on mode.
template <int OP, int MODE>
__device__ __forceinline__ float binary_at(const float* __restrict__ a, const float* __restrict__ b,
                                           size_t e, size_t r, size_t c) {
  float lhs = (MODE == 2) ? a[r] : (MODE == 4) ? a[c] : a[e];
  float rhs = (MODE == 1) ? b[r] : (MODE == 3) ? b[c] : b[e];
  return apply_binary(OP, lhs, rhs);
}

// cols % 4 == 0 and 16-byte aligned full operands: one float4 of the result per step.
template <int OP, int MODE>
__global__ void __launch_bounds__(kThreads)
map_binary_vec(const float* __restrict__ a, const float* __restrict__ b, float4* __restrict__ y,
               size_t nvec, size_t cols) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  const size_t cvec = cols / 4;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < nvec; i += stride) {
    size_t r = i / cvec;
    size_t c = (i - r * cvec) * 4;
    float4 va, vb;
    if (MODE == 2) {
      float s = a[r];
      va = make_float4(s, s, s, s);
    } else if (MODE == 4) {
      va = *reinterpret_cast<const float4*>(a + c);
    } else {
      va = __ldcs(reinterpret_cast<const float4*>(a) + i);
    }
    if (MODE == 1) {
      float s = b[r];
      vb = make_float4(s, s, s, s);
    } else if (MODE == 3) {
      vb = *reinterpret_cast<const float4*>(b + c);
    } else {
      vb = __ldcs(reinterpret_cast<const float4*>(b) + i);
    }
    float4 out;
    out.x = apply_binary(OP, va.x, vb.x);
    out.y = apply_binary(OP, va.y, vb.y);
    out.z = apply_binary(OP, va.z, vb.z);
    out.w = apply_binary(OP, va.w, vb.w);
    __stcs(y + i, out);
  }
}

template <int OP, int MODE>
__global__ void __launch_bounds__(kThreads)
map_binary_scalar(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y,
                  size_t n, size_t cols) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t e = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; e < n; e += stride) {
    size_t r = e / cols;
    size_t c = e - r * cols;
    y[e] = binary_at<OP, MODE>(a, b, e, r, c);
  }
}

struct StridedArgs {
  int rank;
  size_t extent[IB_MAX_RANK];
  ptrdiff_t sa[IB_MAX_RANK];
  ptrdiff_t sb[IB_MAX_RANK];
};

template <int OP, bool BINARY>
__global__ void __launch_bounds__(kThreads)
map_strided(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y,
            size_t n, StridedArgs args) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t e = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; e < n; e += stride) {
    size_t rest = e;
    ptrdiff_t oa = 0, ob = 0;
    for (int d = args.rank - 1; d >= 0; --d) {
      size_t q = rest / args.extent[d];
      size_t coord = rest - q * args.extent[d];
      rest = q;
      oa += static_cast<ptrdiff_t>(coord) * args.sa[d];
      if (BINARY) ob += static_cast<ptrdiff_t>(coord) * args.sb[d];
    }
    y[e] = BINARY ? apply_binary(OP, a[oa], b[ob]) : apply_unary(OP, a[oa]);
  }
}

// The same over four neighbouring results of the innermost axis at a time, for operands that
// are either contiguous along that axis (a 16-byte load) or constant along it (one load): leading
// and middle-axis broadcasts (`bij*bj~bij`), outer products (`i*j~ij`), permutations of leading
// axes (`bij~ibj`).  The index arithmetic, 32-bit here, is paid once per four elements.
// args.extent[rank-1] counts groups of four; the strides of that axis are 4 or 0.
template <int OP, bool BINARY>
__global__ void __launch_bounds__(kThreads)
map_strided_vec(const float* __restrict__ a, const float* __restrict__ b, float4* __restrict__ y,
                unsigned nvec, StridedArgs args, bool a_runs, bool b_runs) {
  const unsigned stride = gridDim.x * kThreads;
  for (unsigned e = blockIdx.x * kThreads + threadIdx.x; e < nvec; e += stride) {
    unsigned rest = e;
    size_t oa = 0, ob = 0;
    for (int d = args.rank - 1; d >= 0; --d) {
      const unsigned ext = static_cast<unsigned>(args.extent[d]);
      const unsigned q = rest / ext;
      const unsigned coord = rest - q * ext;
      rest = q;
      oa += static_cast<size_t>(coord) * static_cast<size_t>(args.sa[d]);
      if (BINARY) ob += static_cast<size_t>(coord) * static_cast<size_t>(args.sb[d]);
    }
    float4 va, vb = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a_runs) {
      va = __ldcs(reinterpret_cast<const float4*>(a + oa));
    } else {
      const float v = __ldg(a + oa);
      va = make_float4(v, v, v, v);
    }
    if (BINARY) {
      if (b_runs) {
        vb = __ldcs(reinterpret_cast<const float4*>(b + ob));
      } else {
        const float v = __ldg(b + ob);
        vb = make_float4(v, v, v, v);
      }
    }
    float4 r;
    r.x = BINARY ? apply_binary(OP, va.x, vb.x) : apply_unary(OP, va.x);
    r.y = BINARY ? apply_binary(OP, va.y, vb.y) : apply_unary(OP, va.y);
    r.z = BINARY ? apply_binary(OP, va.z, vb.z) : apply_unary(OP, va.z);
    r.w = BINARY ? apply_binary(OP, va.w, vb.w) : apply_unary(OP, va.w);
    __stcs(y + e, r);
  }
}

template <int OP>
int launch_unary(const float* x, float* y, size_t n, cudaStream_t s) {
  size_t done = 0;
  if (aligned16(x) && aligned16(y) && n >= 4) {
    size_t nvec = n / 4;
    map_unary_vec<OP><<<grid_for(nvec, kThreads * kVecPerThread), kThreads, 0, s>>>(
        reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), nvec);
    if (int rc = check_launch("ib_map_unary")) return rc;
    done = nvec * 4;
  }
  if (done < n) {
    map_unary_scalar<OP><<<grid_for(n - done, kThreads), kThreads, 0, s>>>(x, y, done, n);
    if (int rc = check_launch("ib_map_unary")) return rc;
  }
  return 0;
}

template <int OP, int MODE>
int launch_binary(const float* a, const float* b, float* y, size_t rows, size_t cols,
                  cudaStream_t s) {
  const size_t n = rows * cols;
  const bool a_full = MODE != 2 && MODE != 4, b_full = MODE != 1 && MODE != 3;
  bool vec = cols % 4 == 0 && aligned16(y) && (!a_full || aligned16(a)) &&
             (!b_full || aligned16(b)) && (MODE != 4 || aligned16(a)) &&
             (MODE != 3 || aligned16(b));
  if (vec) {
    size_t nvec = n / 4;
    map_binary_vec<OP, MODE><<<grid_for(nvec, kThreads), kThreads, 0, s>>>(
        a, b, reinterpret_cast<float4*>(y), nvec, cols);
  } else {
    map_binary_scalar<OP, MODE><<<grid_for(n, kThreads), kThreads, 0, s>>>(a, b, y, n, cols);
  }
  return check_launch("ib_map_binary");
}

template <int OP>
int dispatch_mode(int mode, const float* a, const float* b, float* y, size_t rows, size_t cols,
                  cudaStream_t s) {
  switch (mode) {
    case 0: return launch_binary<OP, 0>(a, b, y, rows, cols, s);
    case 1: return launch_binary<OP, 1>(a, b, y, rows, cols, s);
    case 2: return launch_binary<OP, 2>(a, b, y, rows, cols, s);
    case 3: return launch_binary<OP, 3>(a, b, y, rows, cols, s);
    case 4: return launch_binary<OP, 4>(a, b, y, rows, cols, s);
  }
  return fail("ib_map_binary: mode must be 0..4");
}

// Whether the four-at-a-time form applies: the innermost extent a multiple of four, every operand
// contiguous or constant along it, all other strides and the base pointers keeping 16-byte
// alignment, under 2^32 results and operand elements.
bool strided_vec_ok(const float* a, const float* b, const float* y, size_t n, const StridedArgs& args) {
  if (args.rank < 1 || n >= (1ull << 32) || !aligned16(y)) return false;
  const int in = args.rank - 1;
  if (args.extent[in] % 4 != 0) return false;
  auto operand_ok = [&](const float* p, const ptrdiff_t* st) {
    if (st[in] != 0 && st[in] != 1) return false;
    size_t span = 0;
    for (int d = 0; d < args.rank; ++d) {
      if (st[d] < 0) return false;
      if (st[in] == 1 && d != in && st[d] % 4 != 0) return false;
      span += static_cast<size_t>(st[d]) * (args.extent[d] - 1);
    }
    return span < (1ull << 32) && (st[in] == 0 || aligned16(p));
  };
  return operand_ok(a, args.sa) && (!b || operand_ok(b, args.sb));
}

template <int OP>
int launch_strided(const float* a, const float* b, float* y, size_t n, const StridedArgs& args,
                   cudaStream_t s) {
  if (strided_vec_ok(a, b, y, n, args)) {
    StridedArgs v = args;
    const int in = args.rank - 1;
    const bool a_runs = args.sa[in] == 1, b_runs = b && args.sb[in] == 1;
    v.extent[in] /= 4;
    v.sa[in] *= 4;
    v.sb[in] *= 4;
    const unsigned nvec = static_cast<unsigned>(n / 4);
    if (b)
      map_strided_vec<OP, true><<<grid_for(nvec, kThreads), kThreads, 0, s>>>(
          a, b, reinterpret_cast<float4*>(y), nvec, v, a_runs, b_runs);
    else
      map_strided_vec<OP, false><<<grid_for(nvec, kThreads), kThreads, 0, s>>>(
          a, b, reinterpret_cast<float4*>(y), nvec, v, a_runs, b_runs);
    return check_launch("ib_map_strided");
  }
  if (b)
    map_strided<OP, true><<<grid_for(n, kThreads), kThreads, 0, s>>>(a, b, y, n, args);
  else
    map_strided<OP, false><<<grid_for(n, kThreads), kThreads, 0, s>>>(a, b, y, n, args);
  return check_launch("ib_map_strided");
}


// ---- chains of pointwise operators in one pass ------------------------------------------
//
// `ij-i~ij` then `^ij~ij` then `ij/i~ij` as three launches moves two full-size intermediates
// through memory; here each element is read once, run through the operator list in registers and
// written once.  The operator list is data, not a template: every operator is a warp-uniform switch
// costing two to three instructions per element, which a pass of cheap operators has to spare
// (it stays memory-bound) and one with an exact division and an exponential has not.
// Algorithmic traffic: the operands at their own sizes plus the result, once.
#ifndef IB_CHAIN_BLOCKS
#define IB_CHAIN_BLOCKS 4
#endif
#ifndef IB_CHAIN_VEC
#define IB_CHAIN_VEC 4
#endif
constexpr int kChainVec = IB_CHAIN_VEC;    // float4 results per thread and step

struct ChainArgs {
  int n_ops, n_operands;
  int op[IB_MAX_CHAIN_OPS], lhs[IB_MAX_CHAIN_OPS], rhs[IB_MAX_CHAIN_OPS];
  const float* operand[IB_MAX_CHAIN_OPERANDS];
  int mode[IB_MAX_CHAIN_OPERANDS];   // 0 [r][c], 1 [r], 2 [c], 3 scalar
  bool needs_rc;                     // some operand is per row or per column
  // Row of vector i is umulhi(i, div_mul) >> div_shift (i when a row is one vector wide): exact for
  // i < 2^31 with div_mul = ceil(2^(31+L) / cvec), L = ceil(log2 cvec), div_shift = L - 1.
  unsigned cvec, div_mul, div_shift;
};

// Where a thread's operands come from, for the vectors it holds in one step.  A per-row value or a
// scalar is one number per vector (`scalars`), a full-size or per-column operand four (`vectors`).
// FULL: every vector of the step lies inside the array, so nothing is tested per vector.
template <bool FULL>
struct ChainSource {
  const ChainArgs& a;
  unsigned base, nvec;
  unsigned row[kChainVec];

  __device__ __forceinline__ ChainSource(const ChainArgs& args, unsigned b, unsigned n)
      : a(args), base(b), nvec(n) {
    if (a.needs_rc) {
#pragma unroll
      for (int u = 0; u < kChainVec; ++u) {
        const unsigned i = FULL ? base + u * kThreads : min(base + u * kThreads, nvec - 1);
        row[u] = a.cvec == 1 ? i : __umulhi(i, a.div_mul) >> a.div_shift;
      }
    }
  }
  __device__ __forceinline__ bool live(int u) const { return FULL || base + u * kThreads < nvec; }
  __device__ __forceinline__ bool one_per_vector(int code) const {
    return a.mode[code] == 1 || a.mode[code] == 3;
  }
  __device__ __forceinline__ void scalars(int code, float (&s)[kChainVec]) const {
    const float* p = a.operand[code];
    if (a.mode[code] == 3) {
      const float v = __ldg(p);
#pragma unroll
      for (int u = 0; u < kChainVec; ++u) s[u] = v;
    } else {
#pragma unroll
      for (int u = 0; u < kChainVec; ++u) s[u] = __ldg(p + row[u]);   // row is clamped when !FULL
    }
  }
  __device__ __forceinline__ void vectors(int code, float4 (&dst)[kChainVec]) const {
    const float* p = a.operand[code];
    if (a.mode[code] == 0) {
#pragma unroll
      for (int u = 0; u < kChainVec; ++u)
        if (live(u)) dst[u] = __ldcs(reinterpret_cast<const float4*>(p) + base + u * kThreads);
    } else {
#pragma unroll
      for (int u = 0; u < kChainVec; ++u) {
        const unsigned i = FULL ? base + u * kThreads : min(base + u * kThreads, nvec - 1);
        dst[u] = __ldg(reinterpret_cast<const float4*>(p) + (i - row[u] * a.cvec));
      }
    }
  }
};

// Operators run one after another, so a full-size operand first touched by the third operator
// would add a trip to memory to the thread's critical path.  Its addresses are known up front: ask
// the L2 for them at once (measured on `ij+j`, `>ij`, `ij*ij` at 8192 x 8192: 154 us with, 169
// without).  The same for per-row and per-column vectors measured slower, to L1 or L2, from every
// lane or from one lane per line (`ij-i`, `^ij`: 187 us against 131-145), so those are left to the
// loads themselves.
__device__ __forceinline__ void chain_prefetch_all(const ChainArgs& a, int code, unsigned base,
                                                   unsigned nvec) {
  if (a.mode[code] != 0) return;
  const float4* p = reinterpret_cast<const float4*>(a.operand[code]);
#pragma unroll
  for (int u = 0; u < kChainVec; ++u) {
    unsigned i = base + u * kThreads;
    if (i < nvec) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + i));
  }
}

__device__ __forceinline__ float chain_fetch(const ChainArgs& a, int code, float prev, size_t e,
                                             size_t r, size_t c) {
  if (code == IB_CHAIN_PREV) return prev;
  const float* p = a.operand[code];
  switch (a.mode[code]) {
    case 0: return p[e];
    case 1: return __ldg(p + r);
    case 2: return __ldg(p + c);
    default: return __ldg(p);
  }
}

// The operator list over the sixteen elements a thread holds.  A thread keeps the running result
// and, per operator, the other operand; operator and operand form are decided once per step for
// all sixteen (warp-uniform branches, straight-line arithmetic behind them).  The forms: one
// operand; running value and a vector operand in either order; running value and one number per
// vector in either order (a per-row value is not spread over four registers first).  `src`
// supplies operands: one_per_vector(code), scalars(code, s), vectors(code, t).
enum ChainForm { kUnary, kAccVec, kVecAcc, kAccOne, kOneAcc };

#define IB_CHAIN_LOOP(EXPR)                                        \
  _Pragma("unroll") for (int u = 0; u < kChainVec; ++u) {          \
    float4& A = acc[u];                                            \
    const float4& T = t[u];                                        \
    const float S = one[u];                                        \
    (void)T;                                                       \
    (void)S;                                                       \
    A = EXPR;                                                      \
  }
#define IB_CHAIN_CASE(OP)                                                                          \
  case OP:                                                                                         \
    switch (form) {                                                                                \
      case kUnary:                                                                                 \
        IB_CHAIN_LOOP(make_float4(apply_unary(OP, A.x), apply_unary(OP, A.y), apply_unary(OP, A.z), \
                                  apply_unary(OP, A.w)))                                           \
        break;                                                                                     \
      case kAccVec:                                                                                \
        IB_CHAIN_LOOP(make_float4(apply_binary(OP, A.x, T.x), apply_binary(OP, A.y, T.y),          \
                                  apply_binary(OP, A.z, T.z), apply_binary(OP, A.w, T.w)))         \
        break;                                                                                     \
      case kVecAcc:                                                                                \
        IB_CHAIN_LOOP(make_float4(apply_binary(OP, T.x, A.x), apply_binary(OP, T.y, A.y),          \
                                  apply_binary(OP, T.z, A.z), apply_binary(OP, T.w, A.w)))         \
        break;                                                                                     \
      case kAccOne:                                                                                \
        IB_CHAIN_LOOP(make_float4(apply_binary(OP, A.x, S), apply_binary(OP, A.y, S),              \
                                  apply_binary(OP, A.z, S), apply_binary(OP, A.w, S)))             \
        break;                                                                                     \
      default:                                                                                     \
        IB_CHAIN_LOOP(make_float4(apply_binary(OP, S, A.x), apply_binary(OP, S, A.y),              \
                                  apply_binary(OP, S, A.z), apply_binary(OP, S, A.w)))             \
        break;                                                                                     \
    }                                                                                              \
    break;

template <bool ZERO, class Source>
__device__ __forceinline__ void chain_run(const ChainArgs& a, float4 (&acc)[kChainVec],
                                          const Source& src) {
  if (ZERO) {
#pragma unroll
    for (int u = 0; u < kChainVec; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);   // vectors past the end are not loaded
  }
  if (src.one_per_vector(a.lhs[0])) {
    float first[kChainVec];
    src.scalars(a.lhs[0], first);
#pragma unroll
    for (int u = 0; u < kChainVec; ++u) acc[u] = make_float4(first[u], first[u], first[u], first[u]);
  } else {
    src.vectors(a.lhs[0], acc);
  }
  for (int k = 0; k < a.n_ops; ++k) {
    // The other operand lives for one operator only: declared here, so that nothing but the
    // running value is carried around the loop.
    float4 t[kChainVec];
    float one[kChainVec];
#pragma unroll
    for (int u = 0; u < kChainVec; ++u) {
      t[u] = make_float4(0.f, 0.f, 0.f, 0.f);   // (left unset, the allocator spills four times as much)
      one[u] = 0.0f;
    }
    // Every operator after the first takes the running result on at least one side (the host
    // checks).
    const int lc = a.lhs[k], rc = a.rhs[k];
    const bool acc_left = k == 0 || lc == IB_CHAIN_PREV;
    const int other = acc_left ? rc : lc;
    int form = kUnary;
    if (rc != IB_CHAIN_NONE) {
      if (other == IB_CHAIN_PREV) {
        form = kAccVec;
#pragma unroll
        for (int u = 0; u < kChainVec; ++u) t[u] = acc[u];
      } else if (src.one_per_vector(other)) {
        form = acc_left ? kAccOne : kOneAcc;
        src.scalars(other, one);
      } else {
        form = acc_left ? kAccVec : kVecAcc;
        src.vectors(other, t);
      }
    }
    switch (a.op[k]) {
      IB_CHAIN_CASE(IB_OP_ADD)
      IB_CHAIN_CASE(IB_OP_MUL)
      IB_CHAIN_CASE(IB_OP_SUB)
      IB_CHAIN_CASE(IB_OP_DIV)
      IB_CHAIN_CASE(IB_OP_MAX)
      IB_CHAIN_CASE(IB_OP_MIN)
      IB_CHAIN_CASE(IB_OP_POW)
      IB_CHAIN_CASE(IB_OP_LOG)
      IB_CHAIN_CASE(IB_OP_GT)
      IB_CHAIN_CASE(IB_OP_GE)
      IB_CHAIN_CASE(IB_OP_LT)
      IB_CHAIN_CASE(IB_OP_LE)
      IB_CHAIN_CASE(IB_OP_EQ)
      IB_CHAIN_CASE(IB_OP_NE)
      IB_CHAIN_CASE(IB_OP_AND)
      IB_CHAIN_CASE(IB_OP_OR)
      IB_CHAIN_CASE(IB_OP_XOR)
      IB_CHAIN_CASE(IB_OP_NOT)
    }
  }
}
#undef IB_CHAIN_CASE
#undef IB_CHAIN_LOOP

// cols % 4 == 0, every full or per-column operand 16-byte aligned, under 2^32 elements.  64
// registers, so that four blocks share an SM.
__global__ void __launch_bounds__(kThreads, IB_CHAIN_BLOCKS)
map_chain_vec(const __grid_constant__ ChainArgs a, float4* __restrict__ y, unsigned nvec) {
  // Under 2^30 vectors and at most one block per kThreads * kChainVec of them: 32-bit indexes.
  const unsigned stride = gridDim.x * kThreads * kChainVec;
  for (unsigned base = blockIdx.x * kThreads * kChainVec + threadIdx.x; base < nvec;
       base += stride) {
    for (int e = 0; e < a.n_operands; ++e)
      if (e != a.lhs[0]) chain_prefetch_all(a, e, base, nvec);
    float4 acc[kChainVec];
    if (base + (kChainVec - 1) * kThreads < nvec) {
      chain_run<false>(a, acc, ChainSource<true>(a, base, nvec));
#pragma unroll
      for (int u = 0; u < kChainVec; ++u) __stcs(y + base + u * kThreads, acc[u]);
    } else {
      chain_run<true>(a, acc, ChainSource<false>(a, base, nvec));
#pragma unroll
      for (int u = 0; u < kChainVec; ++u) {
        unsigned i = base + u * kThreads;
        if (i < nvec) __stcs(y + i, acc[u]);
      }
    }
  }
}

// ---- a chain of pointwise operators folded along the rows it produces ----------------------
//
// `ij-i~ij`, `^ij~ij`, `+ij~i` (a softmax's denominator), `ij*ij~ij`-style squares under a sum, a
// mask under an "any": the full-size intermediate never exists.  TPR threads share a row (a warp
// for short rows, the block for long ones); each runs the chain on its vectors and folds them.
// Algorithmic traffic: the operands at their own sizes plus one value per row.
// Operands for the vectors cv, cv + TPR, ... of row r (all of a thread's vectors lie in one row).
template <int TPR>
struct RowSource {
  const ChainArgs& a;
  unsigned r, cv, cvec;
  __device__ __forceinline__ bool one_per_vector(int code) const {
    return a.mode[code] == 1 || a.mode[code] == 3;
  }
  __device__ __forceinline__ void scalars(int code, float (&s)[kChainVec]) const {
    const float* p = a.operand[code];
    const float v = __ldg(a.mode[code] == 1 ? p + r : p);
#pragma unroll
    for (int u = 0; u < kChainVec; ++u) s[u] = v;
  }
  __device__ __forceinline__ void vectors(int code, float4 (&dst)[kChainVec]) const {
    const bool full = a.mode[code] == 0;
    const float4* p4 = reinterpret_cast<const float4*>(a.operand[code]) +
                       (full ? static_cast<size_t>(r) * cvec : 0);
#pragma unroll
    for (int u = 0; u < kChainVec; ++u) {
      const unsigned c = cv + u * TPR;
      if (c < cvec) dst[u] = full ? __ldcs(p4 + c) : __ldg(p4 + c);
    }
  }
};

template <int OP, int TPR>
__global__ void __launch_bounds__(kThreads, IB_CHAIN_BLOCKS)
reduce_chain_vec(const __grid_constant__ ChainArgs a, float* __restrict__ y, unsigned rows,
                 unsigned cvec) {
  constexpr int kRowsPerBlock = kThreads / TPR;
  __shared__ float partial[kThreads / 32];
  const unsigned j = threadIdx.x % TPR;
  for (unsigned r0 = blockIdx.x * kRowsPerBlock; r0 < rows; r0 += gridDim.x * kRowsPerBlock) {
    const unsigned r = r0 + threadIdx.x / TPR;
    const bool live = r < rows;
    float folded = reduce_identity(OP);
    for (unsigned cv = j; live && cv < cvec; cv += TPR * kChainVec) {
      float4 acc[kChainVec];
      chain_run<true>(a, acc, RowSource<TPR>{a, r, cv, cvec});
#pragma unroll
      for (int u = 0; u < kChainVec; ++u)
        if (cv + u * TPR < cvec)
          folded = fold<OP>(folded, fold<OP>(fold<OP>(acc[u].x, acc[u].y), fold<OP>(acc[u].z, acc[u].w)));
    }
    folded = warp_fold<OP>(folded);
    if (TPR == 32) {
      if (j == 0 && live) y[r] = folded;
    } else {
      if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = folded;
      __syncthreads();
      if (threadIdx.x < 32) {
        float v = threadIdx.x < kThreads / 32 ? partial[threadIdx.x] : reduce_identity(OP);
        v = warp_fold<OP>(v);
        if (threadIdx.x == 0 && live) y[r] = v;
      }
      __syncthreads();
    }
  }
}

// Any shape and alignment: one warp per row, one element per lane and step.
template <int OP>
__global__ void __launch_bounds__(kThreads)
reduce_chain_scalar(const __grid_constant__ ChainArgs a, float* __restrict__ y, size_t rows,
                    size_t cols) {
  const int lane = threadIdx.x & 31;
  const size_t warps_total = static_cast<size_t>(gridDim.x) * (kThreads / 32);
  for (size_t r = static_cast<size_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); r < rows;
       r += warps_total) {
    float folded = reduce_identity(OP);
    for (size_t c = lane; c < cols; c += 32) {
      const size_t e = r * cols + c;
      float acc = 0.0f;
      for (int k = 0; k < a.n_ops; ++k) {
        float l = chain_fetch(a, a.lhs[k], acc, e, r, c);
        if (a.rhs[k] != IB_CHAIN_NONE)
          acc = apply_binary(a.op[k], l, chain_fetch(a, a.rhs[k], acc, e, r, c));
        else
          acc = apply_unary(a.op[k], l);
      }
      folded = fold<OP>(folded, acc);
    }
    folded = warp_fold<OP>(folded);
    if (lane == 0) y[r] = folded;
  }
}


__global__ void __launch_bounds__(kThreads)
map_chain_scalar(const __grid_constant__ ChainArgs a, float* __restrict__ y, size_t n,
                 size_t cols) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t e = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; e < n; e += stride) {
    size_t r = 0, c = 0;
    if (a.needs_rc) {
      r = e / cols;
      c = e - r * cols;
    }
    float acc = 0.0f;
    for (int k = 0; k < a.n_ops; ++k) {
      float l = chain_fetch(a, a.lhs[k], acc, e, r, c);
      if (a.rhs[k] != IB_CHAIN_NONE)
        acc = apply_binary(a.op[k], l, chain_fetch(a, a.rhs[k], acc, e, r, c));
      else
        acc = apply_unary(a.op[k], l);
    }
    y[e] = acc;
  }
}
}  // namespace
}  // namespace ib

#define IB_DISPATCH_OP(op, CALL)                                   \
  switch (op) {                                                    \
    case IB_OP_ADD: return CALL(IB_OP_ADD);                        \
    case IB_OP_MUL: return CALL(IB_OP_MUL);                        \
    case IB_OP_SUB: return CALL(IB_OP_SUB);                        \
    case IB_OP_DIV: return CALL(IB_OP_DIV);                        \
    case IB_OP_MAX: return CALL(IB_OP_MAX);                        \
    case IB_OP_MIN: return CALL(IB_OP_MIN);                        \
    case IB_OP_POW: return CALL(IB_OP_POW);                        \
    case IB_OP_LOG: return CALL(IB_OP_LOG);                        \
    case IB_OP_GT: return CALL(IB_OP_GT);                          \
    case IB_OP_GE: return CALL(IB_OP_GE);                          \
    case IB_OP_LT: return CALL(IB_OP_LT);                          \
    case IB_OP_LE: return CALL(IB_OP_LE);                          \
    case IB_OP_EQ: return CALL(IB_OP_EQ);                          \
    case IB_OP_NE: return CALL(IB_OP_NE);                          \
    case IB_OP_AND: return CALL(IB_OP_AND);                        \
    case IB_OP_OR: return CALL(IB_OP_OR);                          \
    case IB_OP_XOR: return CALL(IB_OP_XOR);                        \
    case IB_OP_NOT: return CALL(IB_OP_NOT);                        \
    default: return ib::fail("unknown operator code");             \
  }

extern "C" int ib_map_unary(int op, const float* x, float* y, size_t n, void* stream) {
  if (n == 0) return 0;
  if (!x || !y) return ib::fail("ib_map_unary: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CALL(OP) ib::launch_unary<OP>(x, y, n, s)
  IB_DISPATCH_OP(op, CALL)
#undef CALL
}

extern "C" int ib_map_binary(int op, int mode, const float* a, const float* b, float* y,
                             size_t rows, size_t cols, void* stream) {
  if (rows == 0 || cols == 0) return 0;
  if (!a || !b || !y) return ib::fail("ib_map_binary: null pointer");
  if (op == IB_OP_NOT) return ib::fail("ib_map_binary: operator `!!` has one operand");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CALL(OP) ib::dispatch_mode<OP>(mode, a, b, y, rows, cols, s)
  IB_DISPATCH_OP(op, CALL)
#undef CALL
}

extern "C" int ib_map_strided(int op, const float* a, const float* b, float* y, int rank,
                              const size_t* extent, const ptrdiff_t* stride_a,
                              const ptrdiff_t* stride_b, void* stream) {
  if (rank < 0 || rank > IB_MAX_RANK) return ib::fail("ib_map_strided: rank out of range");
  if (b && op == IB_OP_NOT) return ib::fail("ib_map_strided: operator `!!` has one operand");
  if (!a || !y || (rank > 0 && (!extent || !stride_a)) || (b && rank > 0 && !stride_b))
    return ib::fail("ib_map_strided: null pointer");
  ib::StridedArgs args{};
  args.rank = rank;
  size_t n = 1;
  for (int d = 0; d < rank; ++d) {
    args.extent[d] = extent[d];
    args.sa[d] = stride_a[d];
    args.sb[d] = b ? stride_b[d] : 0;
    n *= extent[d];
  }
  if (n == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CALL(OP) ib::launch_strided<OP>(a, b, y, n, args, s)
  IB_DISPATCH_OP(op, CALL)
#undef CALL
}

namespace ib {
namespace {

// Checks an operator list and fills the kernel's argument block; `vec` says whether the operands
// allow the 16-byte paths (the caller adds its own conditions on the result).
int chain_args(const char* who, int n_ops, const int* ops, int n_operands,
               const float* const* operands, const int* modes, ChainArgs* args, bool* vec) {
  const std::string name(who);
  if (n_ops < 1 || n_ops > IB_MAX_CHAIN_OPS) return fail(name + ": 1 to 8 operators");
  if (n_operands < 1 || n_operands > IB_MAX_CHAIN_OPERANDS) return fail(name + ": 1 to 4 operands");
  if (!ops || !operands || !modes) return fail(name + ": null pointer");
  args->n_ops = n_ops;
  args->n_operands = n_operands;
  for (int e = 0; e < n_operands; ++e) {
    if (!operands[e]) return fail(name + ": null pointer");
    if (modes[e] < 0 || modes[e] > 3) return fail(name + ": operand mode must be 0..3");
    args->operand[e] = operands[e];
    args->mode[e] = modes[e];
    if (modes[e] == 1 || modes[e] == 2) args->needs_rc = true;
    if ((modes[e] == 0 || modes[e] == 2) && !aligned16(operands[e])) *vec = false;
  }
  for (int k = 0; k < n_ops; ++k) {
    const int op = ops[3 * k], lhs = ops[3 * k + 1], rhs = ops[3 * k + 2];
    if (op < IB_OP_ADD || op > IB_OP_NOT) return fail("unknown operator code");
    auto valid = [&](int code, bool may_be_none) {
      if (code == IB_CHAIN_NONE) return may_be_none;
      if (code == IB_CHAIN_PREV) return k > 0;
      return code >= 0 && code < n_operands;
    };
    if (!valid(lhs, false) || !valid(rhs, true)) return fail(name + ": operand code out of range");
    if (op == IB_OP_NOT && rhs != IB_CHAIN_NONE)
      return fail(name + ": operator `!!` has one operand");
    if (k > 0 && lhs != IB_CHAIN_PREV && rhs != IB_CHAIN_PREV)
      return fail(name + ": an operator after the first must take the previous result");
    args->op[k] = op;
    args->lhs[k] = lhs;
    args->rhs[k] = rhs;
  }
  return 0;
}

template <int OP>
int launch_reduce_chain(const ChainArgs& args, bool vec, float* y, size_t rows, size_t cols,
                        cudaStream_t s) {
  const size_t cap = static_cast<size_t>(kNumSMs) * IB_MAP_CAP;
  if (vec && cols >= 4096) {
    reduce_chain_vec<OP, kThreads><<<static_cast<int>(rows < cap ? rows : cap), kThreads, 0, s>>>(
        args, y, static_cast<unsigned>(rows), static_cast<unsigned>(cols / 4));
  } else if (vec) {
    const size_t blocks = (rows + kThreads / 32 - 1) / (kThreads / 32);
    reduce_chain_vec<OP, 32><<<static_cast<int>(blocks < cap ? blocks : cap), kThreads, 0, s>>>(
        args, y, static_cast<unsigned>(rows), static_cast<unsigned>(cols / 4));
  } else {
    const size_t blocks = (rows + kThreads / 32 - 1) / (kThreads / 32);
    reduce_chain_scalar<OP><<<static_cast<int>(blocks < cap ? blocks : cap), kThreads, 0, s>>>(
        args, y, rows, cols);
  }
  return check_launch("ib_reduce_rows_chain");
}

}  // namespace
}  // namespace ib

extern "C" int ib_map_chain(int n_ops, const int* ops, int n_operands, const float* const* operands,
                            const int* modes, float* y, size_t rows, size_t cols, void* stream) {
  ib::ChainArgs args{};
  bool vec = cols % 4 == 0 && ib::aligned16(y) && rows * cols <= 0xffffffffull;
  if (int rc = ib::chain_args("ib_map_chain", n_ops, ops, n_operands, operands, modes, &args, &vec))
    return rc;
  if (rows == 0 || cols == 0) return 0;
  if (!y) return ib::fail("ib_map_chain: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t n = rows * cols;
  if (vec) {
    const size_t nvec = n / 4;
    args.cvec = static_cast<unsigned>(cols / 4);
    if (args.cvec > 1) {
      unsigned log2_ceil = 0;
      while ((1ull << log2_ceil) < args.cvec) ++log2_ceil;
      const unsigned long long two_p = 1ull << (31 + log2_ceil);
      args.div_mul = static_cast<unsigned>((two_p + args.cvec - 1) / args.cvec);
      args.div_shift = log2_ceil - 1;
    }
    ib::map_chain_vec<<<ib::grid_for(nvec, ib::kThreads * ib::kChainVec), ib::kThreads, 0, s>>>(
        args, reinterpret_cast<float4*>(y), static_cast<unsigned>(nvec));
  } else {
    ib::map_chain_scalar<<<ib::grid_for(n, ib::kThreads), ib::kThreads, 0, s>>>(args, y, n, cols);
  }
  return ib::check_launch("ib_map_chain");
}

extern "C" int ib_reduce_rows_chain(int fold_op, int n_ops, const int* ops, int n_operands,
                                    const float* const* operands, const int* modes, float* y,
                                    size_t rows, size_t cols, void* stream) {
  ib::ChainArgs args{};
  bool vec = cols % 4 == 0 && cols > 0 && rows <= 0xffffffffull && rows * cols <= 0xffffffffull;
  if (int rc = ib::chain_args("ib_reduce_rows_chain", n_ops, ops, n_operands, operands, modes, &args,
                              &vec))
    return rc;
  if (rows == 0) return 0;
  if (!y) return ib::fail("ib_reduce_rows_chain: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CALL(OP) ib::launch_reduce_chain<OP>(args, vec, y, rows, cols, s)
  switch (fold_op) {
    case IB_OP_ADD: return CALL(IB_OP_ADD);
    case IB_OP_MUL: return CALL(IB_OP_MUL);
    case IB_OP_MAX: return CALL(IB_OP_MAX);
    case IB_OP_MIN: return CALL(IB_OP_MIN);
    case IB_OP_AND: return CALL(IB_OP_AND);
    case IB_OP_OR: return CALL(IB_OP_OR);
    case IB_OP_XOR: return CALL(IB_OP_XOR);
    default: return ib::fail("operator is not reducible (only + * > < && || ^^ fold)");
  }
#undef CALL
}
