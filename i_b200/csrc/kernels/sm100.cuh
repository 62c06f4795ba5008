// Raw PTX wrappers for the Blackwell (sm_100a) data path: mbarrier, TMA bulk
// tensor copies, tensor memory (TMEM) management, tcgen05 MMA and the matrix /
// instruction descriptors it takes, single-CTA and CTA-pair (cta_group::2) forms.  No load here
// uses cluster multicast or a cta_group qualifier; the one multicast operation is the barrier
// arrival of tcgen05.commit in the CTA-pair GEMM (an arrival, not a data transfer).
//
// Every wait is bounded: a wait that does not complete within kWaitSpinLimit
// polls records a code in a global status word, raises a CTA-wide abort flag
// and returns false, so that a protocol bug surfaces as an error return instead
// of a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace ib {
namespace sm100 {


__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier -------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Shared by all roles of a CTA: set when any wait gives up.
struct AbortState {
  volatile int flag;
};

// Waits for the phase with the given parity.  Returns false (after recording
// `code` in *status and raising the abort flag) when the limit is exceeded or
// another role already aborted.
//
// The limit is a number of polls, not a time: mbarrier.try_wait suspends the
// thread for a hardware-defined interval before it reports "not yet", so
// kWaitSpinLimit polls last from some tens of milliseconds (no suspension at all)
// to a few seconds, and the loop stays a handful of instructions.  That matters: the
// attention kernels run several different instruction streams per SM
// (producers, MMA issuers, statistics and softmax warps) and inline this wait
// at some twenty places; with a clock-based limit (a %globaltimer read, 64-bit
// compares) the waits alone added about 10 KB to what an SM executes per tile,
// and the kernels became bound by instruction fetch.
constexpr uint32_t kWaitSpinLimit = 1u << 22;

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, AbortState* abort,
                                          int* status, int code) {
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (abort->flag) return false;
    if (++spins > kWaitSpinLimit) {
      abort->flag = 1;
      *reinterpret_cast<volatile int*>(status) = code;
      __threadfence_system();
      return false;
    }
  }
  return true;
}

// Whole-warp wait: lane 0 polls, the result is broadcast.  Keeps 31 of 32 lanes
// from hammering the barrier's shared-memory word while the tensor core is
// streaming operands out of the same shared memory.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, AbortState* abort,
                                               int* status, int code) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort, status, code) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  __syncwarp();
  return ok != 0;
}

// ---- programmatic dependent launch ------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may
// start while the kernel before it in the stream is still running.  It must
// execute grid_dependency_wait() before it touches anything that kernel wrote;
// the earlier kernel lets it start early with trigger_dependent_launch() (all of
// its CTAs must have executed that, or exited).  Without the attribute both are
// no-ops.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void trigger_dependent_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Hint: bring [ptr, ptr + bytes) into L2 (16-byte aligned, multiple of 16 bytes).
__device__ __forceinline__ void prefetch_l2_bulk(const void* ptr, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(ptr)),
               "r"(bytes)
               : "memory");
}

// ---- TMA ------------------------------------------------------------------

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// ---- TMEM -----------------------------------------------------------------

// Whole-warp call.  Writes the TMEM base address to *smem_result.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

// Whole-warp call, same warp that allocated.
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 columns: thread i of the warp receives columns [col, col+32) of
// TMEM lane (lane_base + i), where lane_base = 32 * (warp_id % 4) is encoded in
// bits 31:16 of taddr by the caller.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// The same for 16 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// ---- tcgen05.mma ----------------------------------------------------------

enum class Kind { TF32, BF16 };

// 32-bit instruction descriptor for kind::tf32 / kind::f16 with fp32
// accumulation, both operands K-major, no negation, dense.
//   bits 4-5 D format (1 = f32); 7-9 A format; 10-12 B format (tf32 = 2,
//   bf16 = 1); 15/16 A/B major (0 = K); 17-22 N >> 3; 24-28 M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(Kind kind, uint32_t m, uint32_t n) {
  const uint32_t fmt = kind == Kind::TF32 ? 2u : 1u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Operand element formats of the instruction descriptor (A and B take the same one here).
enum class Fmt : uint32_t { F16 = 0, BF16 = 1, TF32 = 2 };
__host__ __device__ constexpr uint32_t make_idesc_fmt(Fmt fmt, uint32_t m, uint32_t n) {
  const uint32_t f = static_cast<uint32_t>(fmt);
  return (1u << 4) | (f << 7) | (f << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// 64-bit shared-memory matrix descriptor for a K-major operand stored as rows
// of 128 bytes with the 128-byte swizzle (what a TMA box of 128 bytes x rows
// with CU_TENSOR_MAP_SWIZZLE_128B writes):
//   bits 0-13 start address >> 4; 16-29 leading byte offset >> 4 (unused for
//   swizzled K-major); 32-45 stride byte offset >> 4 (1024 B between 8-row
//   groups); 46-47 descriptor version (1 on sm_100); 61-63 swizzle mode
//   (2 = 128 B).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  desc |= static_cast<uint64_t>(1) << 16;
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
template <Kind KIND>
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  if (KIND == Kind::TF32) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// D[tmem] (+)= A[tmem] * B[smem]; A is read from tensor memory (rows = lanes).
template <Kind KIND>
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  if (KIND == Kind::TF32) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// The same with the instruction kind chosen by the operand width: 16-bit operands (fp16 or
// bf16, told apart by the descriptor's format field) issue as kind::f16, fp32 ones as kind::tf32.
template <bool HALF>
__device__ __forceinline__ void mma_ts_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  mma_ts<HALF ? Kind::BF16 : Kind::TF32>(d_tmem, a_tmem, b_desc, idesc, accumulate);
}

// Makes `bar` receive one arrival when all MMAs issued so far by this thread
// have completed (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// ---- CTA pairs (cta_group::2) ----------------------------------------------
// Two CTAs of a cluster drive one 256-row MMA: each holds its own 128 rows of A
// and D (same tensor-memory columns in both) and half of the B rows in its own
// shared memory at the same offset.  The even CTA of the pair issues the MMAs.
// Used by the pair GEMM kernel.  Operand loads are plain per-CTA TMA loads (no
// cluster multicast, no cta_group qualifier on a load); only barrier arrivals
// cross between the two CTAs.

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The shared::cluster address of the same shared-memory offset in the cluster's CTA `rank`.
__device__ __forceinline__ uint32_t cluster_addr_of(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}

// The same without a release fence: for a thread that only forwards a signal and has written
// nothing itself (the fence of the releasing form costs such a thread about a thousand cycles per
// arrival, measured).
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_alloc_permit_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

template <Kind KIND>
__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  if (KIND == Kind::TF32) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// One arrival on the barrier at this shared-memory offset in every CTA of
// `cta_mask` once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void mma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}

// mbarrier test whose acquire covers the cluster: for a barrier a peer CTA arrives on.  test_wait
// returns at once (try_wait may suspend the thread for a while first).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Both barriers of a stage in one go (a local one and one a peer arrives on): the two tests are
// issued back to back, so the caller pays one shared-memory round trip, not two.
__device__ __forceinline__ bool mbar_test_both_cluster(uint64_t* a, uint64_t* b, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %3;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 q, [%2], %3;\n\t"
      "and.pred p, p, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_u32(a)), "r"(smem_u32(b)), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ bool mbar_wait_both_cluster(uint64_t* a, uint64_t* b, uint32_t parity,
                                                       AbortState* abort, int* status, int code) {
  uint32_t spins = 0;
  while (!mbar_test_both_cluster(a, b, parity)) {
    if (abort->flag) return false;
    if (++spins > 64u * kWaitSpinLimit) {
      abort->flag = 1;
      *reinterpret_cast<volatile int*>(status) = code;
      __threadfence_system();
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, AbortState* abort,
                                                  int* status, int code) {
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if (abort->flag) return false;
    if (++spins > 64u * kWaitSpinLimit) {        // plain polls: a few tens of cycles each
      abort->flag = 1;
      *reinterpret_cast<volatile int*>(status) = code;
      __threadfence_system();
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace sm100
}  // namespace ib
