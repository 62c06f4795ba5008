// Host-side helpers for the tcgen05 kernels: TMA descriptor encoding (through
// the driver entry point the CUDA runtime hands out, so the library has no
// link-time dependency on libcuda) and the status word bounded waits report to.
#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "sm100.cuh"

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

namespace ib {
namespace {

// mbar_wait with a limit in nanoseconds instead of a number of polls: for this self-test only.
__device__ bool mbar_wait_timed(uint64_t* bar, uint32_t parity, sm100::AbortState* abort, int* status,
                                int code, unsigned long long limit_ns) {
  const unsigned long long start = sm100::global_timer_ns();
  for (;;) {
    if (sm100::mbar_try_wait(bar, parity)) return true;
    if (abort->flag) return false;
    if (sm100::global_timer_ns() - start > limit_ns) {
      abort->flag = 1;
      *reinterpret_cast<volatile int*>(status) = code;
      __threadfence_system();
      return false;
    }
  }
}

// One warp waits on a barrier that nothing ever arrives at, with the limit the caller gives.
// The wait must give up: record its code in the status word, raise the abort flag and return
// false, after which the kernel leaves through its ordinary exit.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ sm100::AbortState abort;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 1);
    abort.flag = 0;
    sm100::fence_barrier_init();
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait_timed(&bar, 0, &abort, status, 250, limit_ns);
  __syncthreads();
  // Every thread sees the flag the waiter raised; a wait that came back "done" would be a bug.
  if (threadIdx.x == 1 && ok && !abort.flag) *reinterpret_cast<volatile int*>(status) = 251;
}

}  // namespace
}  // namespace ib

// Failure detection, exercised without a fault: launches a kernel whose only wait can never be
// satisfied and reports what the host sees afterwards.  The kernels of this library bound every
// device-side wait (sm100.cuh: mbar_wait); a wait that runs out leaves a code in a host-mapped
// status word and the call that synchronises next returns -1 with "a device-side wait timed
// out".  This entry point makes that happen with a wait of `limit_ns` (a millisecond is plenty):
// it returns -1 with that message when the timeout was detected and reported, which is the
// expected outcome, and 0 if the wait did not time out (which would be a defect).  The context
// stays usable; the next launch runs normally.
extern "C" int ib_selftest_wait_timeout(unsigned long long limit_ns, void* stream) {
  using namespace ib;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = device_status_word(s);
  if (!status) return fail("ib_selftest_wait_timeout: cannot allocate the device status word");
  if (limit_ns > 100000000ull) limit_ns = 100000000ull;    // at most 0.1 s
  wait_timeout_selftest_kernel<<<1, 32, 0, s>>>(status, limit_ns);
  cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess)
    return fail(std::string("ib_selftest_wait_timeout: ") + cudaGetErrorString(err));
  count_launch();
  return check_device_status("ib_selftest_wait_timeout", s);
}

// Output assembly across GPUs of one node: queues, on `stream`, one device-to-device copy of
// `bytes` from `src` to each of the `n_dsts` destinations, which are this process's mappings of
// its peers' buffers.  The copies are DMA transfers over NVLink and take no SM from a kernel that
// is running.  `after` (a cudaEvent_t, or null) is waited for first, `done` (a cudaEvent_t, or
// null) is recorded behind the last copy, so a caller's whole publication step is this one call.
// The reference has no counterpart (it runs on one thread of one process).
extern "C" int ib_peer_publish(const void* src, void* const* dsts, int n_dsts, size_t bytes,
                               void* after, void* done, void* stream) {
  using namespace ib;
  if (n_dsts < 0 || (n_dsts > 0 && !dsts)) return fail("ib_peer_publish: no destinations");
  if (bytes > 0 && !src) return fail("ib_peer_publish: null source");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaSuccess;
  if (after) err = cudaStreamWaitEvent(s, static_cast<cudaEvent_t>(after), 0);
  for (int i = 0; err == cudaSuccess && i < n_dsts; ++i) {
    if (!dsts[i]) return fail("ib_peer_publish: null destination");
    if (bytes > 0) err = cudaMemcpyAsync(dsts[i], src, bytes, cudaMemcpyDeviceToDevice, s);
  }
  if (err == cudaSuccess && done) err = cudaEventRecord(static_cast<cudaEvent_t>(done), s);
  if (err != cudaSuccess) return fail(std::string("ib_peer_publish: ") + cudaGetErrorString(err));
  return 0;
}

// The per-device set-up bookkeeping (OncePerDevice), exercised without a GPU: pretends `devices`
// devices each make `calls` calls, the first `failures` set-up attempts on every device failing.
// Returns how many times the set-up function ran: devices * (min(failures, calls) + (calls >
// failures ? 1 : 0)) when every device is set up exactly once after its failures.
extern "C" int ib_selftest_once_per_device(int devices, int calls, int failures) {
  ib::OncePerDevice once;
  int ran = 0;
  int attempts[ib::OncePerDevice::kMaxDevices] = {};
  if (once.run(-1, [] { return 0; }) != -2 ||
      once.run(ib::OncePerDevice::kMaxDevices, [] { return 0; }) != -2)
    return -1;
  for (int c = 0; c < calls; ++c)
    for (int dev = 0; dev < devices && dev < ib::OncePerDevice::kMaxDevices; ++dev)
      once.run(dev, [&] {
        ++ran;
        return attempts[dev]++ < failures ? -1 : 0;
      });
  return ran;
}
