// ib_attention_static: attention for callers that must not allocate.
//
// Some hosts of this library cannot obtain device memory at call time: a
// serving process whose whole GPU budget was handed to another allocator at
// start-up, a real-time loop where a driver allocation's latency is not
// acceptable, or code that runs while allocation is forbidden by its
// framework.  ib_attention needs scratch for the score matrix and expects the
// caller to provide it; this entry point instead keeps that scratch in a
// fixed array that is part of the library image.  The price is a hard size
// limit and no concurrency: see the notes on the function.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace {

// Every GPU that loads the library holds these 32 MiB until the process exits.
constexpr size_t kStaticScratchBytes = IB_ATTENTION_STATIC_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {};

// Device address of the array on the current device.  In host code the array's
// name is only a handle; the address a kernel can use comes from the runtime,
// per device, and is looked up once.
void* scratch_on_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    ib::set_error("ib_attention_static: cannot identify the current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_address[dev]) {
    void* ptr = nullptr;
    cudaError_t rc = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (rc != cudaSuccess || !ptr) {
      ib::set_error(std::string("ib_attention_static: cudaGetSymbolAddress failed: ") +
                    cudaGetErrorString(rc));
      cudaGetLastError();
      return nullptr;
    }
    g_scratch_address[dev] = ptr;
  }
  return g_scratch_address[dev];
}

}  // namespace

extern "C" int ib_attention_static(const float* q, const float* k, const float* v, float* o,
                                   size_t batch, size_t nq, size_t nk, size_t d, size_t dv,
                                   int v_kmajor, void* stream) {
  const size_t need =
      ib_attention_workspace_bytes(batch, nq, nk, d, dv, v_kmajor, IB_PRECISION_FP32);
  if (need == SIZE_MAX)
    return ib::fail("ib_attention_static: extents too large (an element count does not fit size_t)");
  if (need > kStaticScratchBytes)
    return ib::fail("ib_attention_static: batch*nq*nk = " + std::to_string(batch * nq * nk) +
                    " scores need " + std::to_string(need) + " bytes of scratch, the built-in " +
                    "array holds " + std::to_string(kStaticScratchBytes) +
                    "; use ib_attention with a caller workspace");
  void* scratch = scratch_on_current_device();
  if (!scratch) return -1;
  // Nothing in the scratch has to start at zero: the first contraction writes
  // every score the later steps read.
  return ib_attention(q, k, v, o, batch, nq, nk, d, dv, v_kmajor, IB_PRECISION_FP32, 0, scratch,
                      kStaticScratchBytes, stream);
}
