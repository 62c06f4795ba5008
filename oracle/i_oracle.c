/*
 * CPU oracle for the i component hot path.  TEST INFRASTRUCTURE ONLY: nothing
 * in the shipped library links, imports or calls this file; the parity tests,
 * the smoke check and the CPU-baseline leg of the benchmark are its only users.
 *
 * Every function restates, in plain scalar C, the arithmetic the reference's C
 * backend emits for one kind of component ("restated, not emitted": the
 * reference's compiler is Rust and cannot be built where this runs).  The rules
 * followed, by reference file:
 *   - tile loops ceil(N/F) with inner guards `tile*F + inner < N`
 *       compiler/src/lower/exec_plan_to_module.rs:303-335, 541-557
 *   - reduction identities (+ 0, * 1, > -inf, < +inf)      ...:592-603
 *   - unary defaults (-x = 0-x, /x = 1/x, ^x = powf(e32,x), $x = logf(x),
 *     >x = fmaxf(0,x), <x = fminf(0,x))                    ...:605-640
 *   - op spelling (separate mul/add, fmaxf, fminf, powf, logf; binary `$`
 *     drops its second operand)     compiler/src/backends/c/expr.rs:127-148, 319-321
 *   - the literal e prints as 2.71828175f                  compiler/src/backends/c/expr.rs:350-366
 *   - fused attention kernel                               ilang-python/annotated-flashattn.c:52-310
 *
 * Parity pin: io_attention_fused is checked bit-for-bit against the reference's
 * own emitted C (ilang-python/annotated-flashattn.c, built by oracle/Makefile
 * into oracle/_ref/) and all functions against float64 NumPy on the cases of
 * ilang-python/test.py and ilang-python/flash-attn.py; the reference holds no
 * numeric golden vectors.
 *
 * Build exactly as the reference builds generated code (core/src/lib.rs:400-407):
 *   cc -O3 -shared -fPIC i_oracle.c -o libi_oracle.so -lm
 * i.e. no -ffast-math and no -march, so float sums stay in strict ascending
 * order with separate multiply and add.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>

#define IO_E 2.71828175f

enum {
  IO_ADD = 0, IO_MUL = 1, IO_SUB = 2, IO_DIV = 3,
  IO_MAX = 4, IO_MIN = 5, IO_POW = 6, IO_LOG = 7,
  /* comparisons and logic: C operators on floats, the int result stored as 0.0f / 1.0f
   * (compiler/src/backends/c/expr.rs:136-146, xor at :331-339) */
  IO_GT = 8, IO_GE = 9, IO_LT = 10, IO_LE = 11, IO_EQ = 12, IO_NE = 13,
  IO_AND = 14, IO_OR = 15, IO_XOR = 16, IO_NOT = 17
};

static inline size_t io_ceil_div(size_t n, size_t f) { return (n + f - 1) / f; }

static inline float io_binary(int op, float a, float b) {
  switch (op) {
    case IO_ADD: return a + b;
    case IO_MUL: return a * b;
    case IO_SUB: return a - b;
    case IO_DIV: return a / b;
    case IO_MAX: return fmaxf(a, b);
    case IO_MIN: return fminf(a, b);
    case IO_POW: return powf(a, b);
    case IO_LOG: return logf(a); /* second operand dropped by the C backend */
    case IO_GT: return (float)(a > b);
    case IO_GE: return (float)(a >= b);
    case IO_LT: return (float)(a < b);
    case IO_LE: return (float)(a <= b);
    case IO_EQ: return (float)(a == b);
    case IO_NE: return (float)(a != b);
    case IO_AND: return (float)(a && b);
    case IO_OR: return (float)(a || b);
    case IO_XOR: return (float)(((a) != 0.0f) != ((b) != 0.0f));
  }
  return NAN;
}

static inline float io_unary(int op, float x) {
  switch (op) {
    case IO_ADD: case IO_MUL: return x;
    case IO_SUB: return 0.0f - x;
    case IO_DIV: return 1.0f / x;
    case IO_MAX: return fmaxf(0.0f, x);
    case IO_MIN: return fminf(0.0f, x);
    case IO_POW: return powf(IO_E, x);
    case IO_LOG: return logf(x);
    /* unary forms, compiler/src/lower/exec_plan_to_module.rs:613-637: comparisons
     * compare with 0.0f, and / or / xor copy their operand, not is `!x` */
    case IO_GT: return (float)(x > 0.0f);
    case IO_GE: return (float)(x >= 0.0f);
    case IO_LT: return (float)(x < 0.0f);
    case IO_LE: return (float)(x <= 0.0f);
    case IO_EQ: return (float)(x == 0.0f);
    case IO_NE: return (float)(x != 0.0f);
    case IO_AND: case IO_OR: case IO_XOR: return x;
    case IO_NOT: return (float)(!x);
  }
  return NAN;
}

static inline float io_identity(int op) {
  switch (op) {
    case IO_ADD: return 0.0f;
    case IO_MUL: return 1.0f;
    case IO_MAX: return -INFINITY;
    case IO_MIN: return INFINITY;
    case IO_AND: return 1.0f;   /* exec_plan_to_module.rs:592-603 */
    case IO_OR: case IO_XOR: return 0.0f;
  }
  return NAN;
}

/* y[r][c] = op(x[r][c]); unary map over a row-major rows x cols view. */
void io_map_unary(int op, const float* x, float* y, size_t n) {
  for (size_t i = 0; i < n; ++i) y[i] = io_unary(op, x[i]);
}

/*
 * Binary pointwise map with broadcast, y[r][c] = op(a, b).
 * mode 0: a[r][c] op b[r][c]; mode 1: a[r][c] op b[r] (`ij-i~ij`);
 * mode 2: a[r] op b[r][c]; mode 3: a[r][c] op b[c]; mode 4: a[c] op b[r][c].
 */
void io_map_binary(int op, int mode, const float* a, const float* b, float* y,
                   size_t rows, size_t cols) {
  for (size_t r = 0; r < rows; ++r) {
    for (size_t c = 0; c < cols; ++c) {
      size_t e = r * cols + c;
      float lhs = (mode == 2) ? a[r] : (mode == 4) ? a[c] : a[e];
      float rhs = (mode == 1) ? b[r] : (mode == 3) ? b[c] : b[e];
      y[e] = io_binary(op, lhs, rhs);
    }
  }
}

/*
 * Row reduction y[r] = fold op over ascending c of x[r][c], starting from the
 * op's identity (default index-major order: ilang-python/test.py:109-128).
 */
void io_reduce_rows(int op, const float* x, float* y, size_t rows, size_t cols) {
  for (size_t r = 0; r < rows; ++r) {
    float acc = io_identity(op);
    for (size_t c = 0; c < cols; ++c) acc = io_binary(op, acc, x[r * cols + c]);
    y[r] = acc;
  }
}

/*
 * Contraction C[i][j] = sum_k A(i,k) * B(j,k), product then add, ascending k,
 * accumulator zero-initialised per output element.  a_kmajor / b_kmajor pick
 * the operand layouts: 1 = [row][k] (as `ik*jk~ijk`), 0 = [k][row] (as the
 * second operand of `ij*jk~ikj`).  Tiled 16x16 in (j-tile, i-tile) order like
 * the README schedule `jii'j'k`; the per-element arithmetic does not depend on
 * the tile order.
 */
void io_contract(const float* A, const float* B, float* C, size_t ni, size_t nj,
                 size_t nk, int a_kmajor, int b_kmajor) {
  for (size_t jt = 0; jt < io_ceil_div(nj, 16); ++jt)
    for (size_t it = 0; it < io_ceil_div(ni, 16); ++it)
      for (size_t ii = 0; ii < 16; ++ii) {
        size_t i = it * 16 + ii;
        if (i >= ni) continue;
        for (size_t jj = 0; jj < 16; ++jj) {
          size_t j = jt * 16 + jj;
          if (j >= nj) continue;
          float acc = 0.0f;
          for (size_t k = 0; k < nk; ++k) {
            float a = a_kmajor ? A[i * nk + k] : A[k * ni + i];
            float b = b_kmajor ? B[j * nk + k] : B[k * nj + j];
            float prod = a * b;
            acc = acc + prod;
          }
          C[i * nj + j] = acc;
        }
      }
}

/*
 * Row softmax as the three naive kernels of ilang-python/flash-attn.py:60-62
 * produce it: m = fold fmaxf from -inf; y = x - m; e = powf(e32, y);
 * l = ascending fp32 sum of e from 0; out = e / l.
 */
void io_row_softmax(const float* x, float* out, size_t rows, size_t cols) {
  for (size_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float* yr = out + r * cols;
    float m = -INFINITY;
    for (size_t c = 0; c < cols; ++c) m = fmaxf(m, xr[c]);
    float l = 0.0f;
    for (size_t c = 0; c < cols; ++c) {
      float e = powf(IO_E, xr[c] - m);
      yr[c] = e;
      l = l + e;
    }
    for (size_t c = 0; c < cols; ++c) yr[c] = yr[c] / l;
  }
}

/*
 * Fused online-softmax attention O = softmax(Q K^T) V with 16-wide KV tiles,
 * following ilang-python/annotated-flashattn.c:52-310 step by step per row:
 * per KV tile (ascending): s = Q.K (ascending d), m_old = m, m = fold fmaxf,
 * p = powf(e32, s - m), l_old = l, l = l * powf(e32, m_old - m) then + p
 * (ascending), p = p / l, O = O * powf(e32, m_old - m), O = O * (l_old / l),
 * O = 0 on the first tile, O = O + p * V (ascending j within the tile).
 * Rows are independent, so this runs row by row rather than in 16-row tiles.
 * Q is nq x d, K is nk x d, V is nk x dv, O is nq x dv, all row-major.
 */
void io_attention_fused(const float* Q, const float* K, const float* V, float* O,
                        size_t nq, size_t nk, size_t d, size_t dv) {
  float s[16], p[16];
  for (size_t i = 0; i < nq; ++i) {
    float m = -INFINITY, l = 0.0f;
    float* o = O + i * dv;
    const float* q = Q + i * d;
    for (size_t jt = 0; jt < io_ceil_div(nk, 16); ++jt) {
      size_t w = nk - jt * 16 < 16 ? nk - jt * 16 : 16;
      for (size_t jj = 0; jj < w; ++jj) {
        const float* kr = K + (jt * 16 + jj) * d;
        float acc = 0.0f;
        for (size_t c = 0; c < d; ++c) {
          float prod = q[c] * kr[c];
          acc = acc + prod;
        }
        s[jj] = acc;
      }
      float m_old = m;
      for (size_t jj = 0; jj < w; ++jj) m = fmaxf(m, s[jj]);
      for (size_t jj = 0; jj < w; ++jj) p[jj] = powf(IO_E, s[jj] - m);
      float l_old = l;
      l = l * powf(IO_E, m_old - m);
      for (size_t jj = 0; jj < w; ++jj) l = l + p[jj];
      for (size_t jj = 0; jj < w; ++jj) p[jj] = p[jj] / l;
      float shift = powf(IO_E, m_old - m);
      float ratio = l_old / l;
      for (size_t c = 0; c < dv; ++c) {
        float acc = (o[c] * shift) * ratio;
        if (jt == 0) acc = 0.0f;
        for (size_t jj = 0; jj < w; ++jj) {
          float prod = p[jj] * V[(jt * 16 + jj) * dv + c];
          acc = acc + prod;
        }
        o[c] = acc;
      }
    }
  }
}

/*
 * Unfused attention as the five-kernel naive schedule computes it
 * (ilang-python/flash-attn.py:57-65): S = Q K^T, row softmax, P V.
 * scratch holds nq*nk floats.
 */
void io_attention_naive(const float* Q, const float* K, const float* V, float* O,
                        float* scratch, size_t nq, size_t nk, size_t d, size_t dv) {
  io_contract(Q, K, scratch, nq, nk, d, 1, 1);
  io_row_softmax(scratch, scratch, nq, nk);
  io_contract(scratch, V, O, nq, dv, nk, 1, 0);
}
