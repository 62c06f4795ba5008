// Host-side helpers for the tcgen05 kernels: TMA descriptor encoding (through
// the driver entry point the CUDA runtime hands out, so the library has no
// link-time dependency on libcuda) and the status word bounded waits report to.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace ib {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult query;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault,
                                              &query);
    if (err != cudaSuccess || query != cudaDriverEntryPointSuccess) return EncodeTiledFn(nullptr);
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

constexpr int kMaxDevices = 64;
std::mutex g_status_mutex;
int* g_status_host[kMaxDevices] = {};
int* g_status_dev[kMaxDevices] = {};

}  // namespace

int make_tensor_map_f32(CUtensorMap* map, const float* base, size_t batch, size_t rows,
                        size_t cols, size_t row_pitch, size_t batch_pitch, unsigned box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return fail("cuTensorMapEncodeTiled is not available from this CUDA driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || (row_pitch * 4) % 16 || (batch_pitch * 4) % 16)
    return fail("tensor map: base and pitches must be 16-byte aligned");
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {row_pitch * sizeof(float), batch_pitch * sizeof(float)};
  cuuint32_t box[3] = {32, box_rows, 1};
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims,
                   strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return fail("cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(rc)));
  return 0;
}

int make_tensor_map_bf16(CUtensorMap* map, const void* base, size_t batch, size_t rows,
                         size_t cols, size_t row_pitch, size_t batch_pitch, unsigned box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return fail("cuTensorMapEncodeTiled is not available from this CUDA driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || (row_pitch * 2) % 16 || (batch_pitch * 2) % 16)
    return fail("tensor map: base and pitches must be 16-byte aligned");
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {row_pitch * 2, batch_pitch * 2};
  cuuint32_t box[3] = {64, box_rows, 1};          // 64 bf16 = one 128-byte swizzled row
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims,
                   strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return fail("cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(rc)));
  return 0;
}

int* device_status_word(cudaStream_t) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status_dev[dev]) {
    int* host = nullptr;
    if (cudaHostAlloc(&host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) return nullptr;
    *host = 0;
    int* devptr = nullptr;
    if (cudaHostGetDevicePointer(&devptr, host, 0) != cudaSuccess) return nullptr;
    g_status_host[dev] = host;
    g_status_dev[dev] = devptr;
  }
  return g_status_dev[dev];
}

int check_device_status(const char* what, cudaStream_t) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  int code = 0;
  {
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status_host[dev]) return 0;
    code = *static_cast<volatile int*>(g_status_host[dev]);
    if (code) *static_cast<volatile int*>(g_status_host[dev]) = 0;
  }
  if (code)
    return fail(std::string(what) + ": a device-side wait timed out (code " +
                std::to_string(code) + "); results of that launch are invalid");
  return 0;
}

}  // namespace ib

// Undocumented hook for kernel development: returns and clears the code a bounded
// device-side wait left for the current device, 0 if none.
extern "C" int ib_debug_take_device_status(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= ib::kMaxDevices) return 0;
  std::lock_guard<std::mutex> lock(ib::g_status_mutex);
  if (!ib::g_status_host[dev]) return 0;
  const int code = *static_cast<volatile int*>(ib::g_status_host[dev]);
  *static_cast<volatile int*>(ib::g_status_host[dev]) = 0;
  return code;
}
