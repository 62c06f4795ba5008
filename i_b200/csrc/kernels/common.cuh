// Shared device helpers and host-side launch bookkeeping for the ib_* kernels.
#pragma once

#include <cuda_runtime.h>
#include <math_constants.h>

#include <cstddef>
#include <cstdint>
#include <mutex>
#include <string>

#include "i_b200.h"

namespace ib {

// Implemented in core/runtime.cc: records the thread-local message i_error() returns.
void set_error(const std::string& message);
// Bumps the counter behind i_b200_launch_count().
void count_launch(size_t n = 1);

inline int fail(const std::string& message) {
  set_error(message);
  return -1;
}

inline int check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(std::string(what) + ": " + cudaGetErrorString(err));
  count_launch();
  return 0;
}

constexpr int kNumSMs = 148;  // B200

// Set-up that has to happen once per device and per kernel (function attributes such as the
// opt-in to more than 48 KB of dynamic shared memory belong to the device's context, not to the
// process): run(device, f) calls f the first time it sees `device` and remembers success.  A
// failed f is tried again on the next call.  Safe to call from several threads.
class OncePerDevice {
 public:
  static constexpr int kMaxDevices = 64;
  // Returns f's result (0 = ok) on the first call for a device, 0 afterwards, -2 for a device
  // number outside [0, kMaxDevices).
  template <typename F>
  int run(int device, F&& f) {
    if (device < 0 || device >= kMaxDevices) return -2;
    std::lock_guard<std::mutex> lock(mutex_);
    if (done_[device]) return 0;
    const int rc = f();
    if (rc == 0) done_[device] = true;
    return rc;
  }

 private:
  std::mutex mutex_;
  bool done_[kMaxDevices] = {};
};

// powf(2.71828175f, x), the reference C backend's exp
// (compiler/src/backends/c/expr.rs:350-366 prints e as 2.71828175f).  x*log2(e32)
// is carried as a two-float product so the result stays within a few ulp of the
// libm value over the whole range a softmax sees.
__device__ __forceinline__ float exp_e32(float x) {
  const float l_hi = 1.4426950216293335f;      // fp32(log2(2.71828175))
  const float l_lo = -2.4551930266625277e-08f; // log2(2.71828175) - l_hi
  if (!(fabsf(x) < 200.0f)) return x > 0.0f ? CUDART_INF_F : (x < 0.0f ? 0.0f : x);
  float hi = x * l_hi;
  float lo = fmaf(x, l_lo, fmaf(x, l_hi, -hi));
  float n = rintf(hi);
  float f = (hi - n) + lo;
  return ldexpf(exp2f(f), static_cast<int>(n));
}

// Same function with the range reduction done by hand: 2^f from the MUFU
// (ex2.approx, ~2 ulp) and 2^n added into the exponent field.  Results that
// would be subnormal, overflow, or come from inf/NaN take the exact path.
__device__ __forceinline__ float exp_e32_fast(float x) {
  const float l_hi = 1.4426950216293335f;
  const float l_lo = -2.4551930266625277e-08f;
  const float magic = 12582912.0f;             // 1.5 * 2^23: adding it rounds to the nearest integer
  float hi = x * l_hi;
  float lo = fmaf(x, l_lo, fmaf(x, l_hi, -hi));
  if (!(fabsf(hi) < 125.0f)) return exp_e32(x);   // subnormal or overflowing results, inf, NaN
  float shifted = hi + magic;                  // integer part now sits in the low mantissa bits
  float n = shifted - magic;
  float f = (hi - n) + lo;
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(f));
  // 2^n: add n to the exponent field (the low bits of `shifted` are n in two's complement).
  return __int_as_float(__float_as_int(r) + (__float_as_int(shifted) << 23));
}

__device__ __forceinline__ float apply_binary(int op, float a, float b) {
  switch (op) {
    case IB_OP_ADD: return a + b;
    case IB_OP_MUL: return a * b;
    case IB_OP_SUB: return a - b;
    case IB_OP_DIV: return a / b;
    case IB_OP_MAX: return fmaxf(a, b);
    case IB_OP_MIN: return fminf(a, b);
    case IB_OP_POW: return powf(a, b);
    case IB_OP_GT: return a > b ? 1.0f : 0.0f;
    case IB_OP_GE: return a >= b ? 1.0f : 0.0f;
    case IB_OP_LT: return a < b ? 1.0f : 0.0f;
    case IB_OP_LE: return a <= b ? 1.0f : 0.0f;
    case IB_OP_EQ: return a == b ? 1.0f : 0.0f;
    case IB_OP_NE: return a != b ? 1.0f : 0.0f;
    case IB_OP_AND: return (a != 0.0f && b != 0.0f) ? 1.0f : 0.0f;
    case IB_OP_OR: return (a != 0.0f || b != 0.0f) ? 1.0f : 0.0f;
    case IB_OP_XOR: return ((a != 0.0f) != (b != 0.0f)) ? 1.0f : 0.0f;
    default: return logf(a);  // IB_OP_LOG: the C backend drops the second operand
  }
}

__device__ __forceinline__ float apply_unary(int op, float x) {
  switch (op) {
    case IB_OP_ADD:
    case IB_OP_MUL: return x;
    case IB_OP_SUB: return 0.0f - x;
    case IB_OP_DIV: return 1.0f / x;
    case IB_OP_MAX: return fmaxf(0.0f, x);
    case IB_OP_MIN: return fminf(0.0f, x);
    case IB_OP_POW: return exp_e32_fast(x);
    case IB_OP_GT: return x > 0.0f ? 1.0f : 0.0f;
    case IB_OP_GE: return x >= 0.0f ? 1.0f : 0.0f;
    case IB_OP_LT: return x < 0.0f ? 1.0f : 0.0f;
    case IB_OP_LE: return x <= 0.0f ? 1.0f : 0.0f;
    case IB_OP_EQ: return x == 0.0f ? 1.0f : 0.0f;
    case IB_OP_NE: return x != 0.0f ? 1.0f : 0.0f;
    case IB_OP_AND:
    case IB_OP_OR:
    case IB_OP_XOR: return x;
    case IB_OP_NOT: return x == 0.0f ? 1.0f : 0.0f;
    default: return logf(x);
  }
}

__device__ __forceinline__ float reduce_identity(int op) {
  switch (op) {
    case IB_OP_ADD: return 0.0f;
    case IB_OP_MUL: return 1.0f;
    case IB_OP_MAX: return -CUDART_INF_F;
    case IB_OP_AND: return 1.0f;
    case IB_OP_OR:
    case IB_OP_XOR: return 0.0f;
    default: return CUDART_INF_F;  // IB_OP_MIN
  }
}

template <int OP>
__device__ __forceinline__ float fold(float a, float b) {
  if (OP == IB_OP_ADD) return a + b;
  if (OP == IB_OP_MUL) return a * b;
  if (OP == IB_OP_MAX) return fmaxf(a, b);
  if (OP == IB_OP_MIN) return fminf(a, b);
  // Logic folds work on truth values; every element passes through at least one
  // fold with the identity, so results are always 0 or 1 as in the serial form.
  return apply_binary(OP, a, b);
}

template <int OP>
__device__ __forceinline__ float warp_fold(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = fold<OP>(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace ib
