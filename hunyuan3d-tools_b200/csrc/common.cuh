// Shared device helpers for the sm_100a W8A8 kernels: mbarrier, TMA, tcgen05 wrappers
// (inline PTX), bounded waits and the descriptor encodings used by every GEMM here.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/hy3d_int8.h"

#define HY3D_ABI_VERSION 201

namespace hy3d {

// ------------------------------------------------------------------------------------
// Device-side error word.  A kernel whose bounded wait runs out stores a code here and
// leaves through its normal teardown, so the context stays usable.  The library is built
// as one translation unit (hy3d_int8.cu includes every kernel file), so this is the single
// definition.
// ------------------------------------------------------------------------------------
__device__ int g_device_status = 0;

// Optional timeline tracing of one CTA (compiled in only with -DHY3D_TRACE; never part of
// the shipped library).  Each record: SM clock << 16 | event << 8 | argument.
#ifdef HY3D_TRACE
__device__ unsigned long long g_trace_buf[4 * 4096];
__device__ int g_trace_cta = 0;
// Store-only (no atomics, nothing to wait for): every role keeps its own record counter
// in a register and owns a 4096-entry slice of the buffer.
__device__ __forceinline__ void trace_event(int role, unsigned& idx, int ev, int arg) {
  if (idx < 4096u)
    g_trace_buf[role * 4096 + idx] = (static_cast<unsigned long long>(clock64()) << 16) |
                                     (static_cast<unsigned long long>(ev & 0xFF) << 8) | (arg & 0xFF);
  ++idx;
}
#define HY3D_TRACE_DECL(name) unsigned name = (static_cast<int>(blockIdx.x) == g_trace_cta) ? 0u : 4096u
#define HY3D_CLK() clock64()
#define HY3D_TRACE_RAW(slot, value) do { if (static_cast<int>(blockIdx.x) == g_trace_cta) g_trace_buf[3 * 4096 + (slot)] = (value); } while (0)
#define HY3D_TRACE_EVENT(role, idx, ev, arg) trace_event(role, idx, ev, arg)
#ifdef HY3D_TRACE_PER_STAGE
#define HY3D_TRACE_FINE(role, idx, ev, arg) trace_event(role, idx, ev, arg)
#else
#define HY3D_TRACE_FINE(role, idx, ev, arg) ((void)0)
#endif
#else
#define HY3D_TRACE_DECL(name) ((void)0)
#define HY3D_CLK() 0ll
#define HY3D_TRACE_RAW(slot, value) ((void)0)
#define HY3D_TRACE_EVENT(role, idx, ev, arg) ((void)0)
#define HY3D_TRACE_FINE(role, idx, ev, arg) ((void)0)
#endif

enum DeviceError : int {
  kDevOk = 0,
  kDevTimeoutFull = 101,       // consumer gave up waiting for a TMA stage
  kDevTimeoutEmpty = 102,      // producer gave up waiting for a free stage
  kDevTimeoutTmemFull = 103,   // epilogue gave up waiting for the accumulators
  kDevTimeoutTmemEmpty = 104,  // MMA issuer gave up waiting for a drained accumulator
  kDevTimeoutStore = 105,
  kDevTimeoutPeer = 106,       // CTA-pair handshake
  kDevBadAlignment = 107,      // dynamic shared memory not 1024-byte aligned
  kDevTimeoutQuant = 108,      // producer gave up waiting for a tile of the fused quantiser
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------------------------
// Programmatic dependent launch: a kernel launched with the programmatic-serialisation
// attribute may start while its predecessor in the stream is still running; everything
// before pdl_wait() (barrier set-up, tensor-memory allocation, descriptor prefetch) overlaps
// with the predecessor's tail, everything after it sees the predecessor's memory complete.
// Without the launch attribute both are no-ops.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `cta_rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta_rank) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
      ::"r"(bar), "r"(cta_rank)
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking probe.  try_wait may park the thread and was measured to hand control back
// only a few hundred nanoseconds after the phase completes; polling with test_wait reacts
// within tens of cycles, which matters for the per-stage handshakes of the GEMM pipelines.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Upper bound on any single wait.  Far above every legitimate wait of these kernels
// (whole launches last well under 10 ms) and short enough that a protocol error ends the
// kernel instead of hanging the device.
constexpr uint64_t kWaitLimitNs = 2000ull * 1000ull * 1000ull;
// The limit in force; tests shorten it to a few milliseconds (hy3d_set_wait_limit_ns).
__device__ unsigned long long g_wait_limit_ns = kWaitLimitNs;

// Bounded wait.  `abort_flag` lives in shared memory and is set by whichever role times
// out first, so the other roles leave their waits promptly.  Returns false on give-up.
// Bounded wait.  `abort_flag` lives in shared memory and is set by whichever role times
// out first, so the other roles leave their waits promptly.  Returns false on give-up.
// kSpin selects test_wait polling (lowest wake-up latency) instead of the parking try_wait.
template <bool kSpin = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int err_code) {
  if (kSpin ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (kSpin ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
    if ((++spins & (kSpin ? 0xFFFu : 0xFFu)) == 0) {
      if (*abort_flag) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > g_wait_limit_ns) {
        *abort_flag = 1;
        atomicCAS(&g_device_status, 0, err_code);
        return false;
      }
    }
  }
}

// Exercises the give-up path of the bounded wait without disturbing anything else: one thread
// waits on an mbarrier that nobody will ever arrive on; once the limit in force runs out it
// records kDevTimeoutFull in the device status word and the kernel returns normally.
__global__ void wait_selftest_kernel() {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
    mbar_wait(smem_u32(&bar), 0, &abort_flag, kDevTimeoutFull);
    mbar_inval(smem_u32(&bar));
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies; never multicast)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// CTA-pair form: the data lands in this CTA's shared memory, the completion bytes are
// credited to `bar_cluster`, a shared::cluster address that may name the pair's other CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m,
                                                 uint32_t bar_cluster, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int32_t x,
                                             int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int kPending>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
template <int kPending>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}

// ------------------------------------------------------------------------------------
// tcgen05: tensor memory, MMA issue, commit, loads
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc_1cta(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_1cta() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_1cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// One dense int8 MMA: D[tmem] (+)= A[smem] * B[smem]^T.
__device__ __forceinline__ void mma_i8_1cta(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_i8_2cta(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same instructions with each descriptor given as (low word, shared high word): the
// issuing thread then advances a 32-bit address field instead of doing 64-bit arithmetic.
template <int kG>
__device__ __forceinline__ void mma_i8_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                            uint32_t desc_hi, uint32_t idesc, uint32_t accumulate) {
  if (kG == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// One 2:4-sparse int8 MMA: A compressed in smem, its metadata at e_tmem.
__device__ __forceinline__ void mma_sp_i8_1cta(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b,
                                               uint32_t e_tmem, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.sp.cta_group::1.kind::i8 [%0], %1, %2, [%3], %4, p;\n\t}"
      ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(e_tmem), "r"(idesc), "r"(accumulate)
      : "memory");
}
// CTA-pair forms: A is 256 rows (128 per CTA), B is split by columns between the CTAs, each
// CTA's metadata sits in its own tensor memory.
__device__ __forceinline__ void mma_sp_i8_2cta(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b,
                                               uint32_t e_tmem, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.sp.cta_group::2.kind::i8 [%0], %1, %2, [%3], %4, p;\n\t}"
      ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(e_tmem), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_cp_128x128b_2cta(uint32_t dst_tmem, uint64_t src_desc) {
  asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(dst_tmem), "l"(src_desc)
               : "memory");
}
// Shared memory -> tensor memory copy of 128 lanes x 128 bits (sparse metadata).
__device__ __forceinline__ void tmem_cp_128x128b_1cta(uint32_t dst_tmem, uint64_t src_desc) {
  asm volatile("tcgen05.cp.cta_group::1.128x128b [%0], %1;" ::"r"(dst_tmem), "l"(src_desc)
               : "memory");
}
// Makes `bar` complete one arrival once every tcgen05 operation issued so far by this
// thread has finished.
__device__ __forceinline__ void tc_commit_1cta(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar) : "memory");
}
// CTA-pair form: arrives on the barrier at this offset in each CTA named by `cta_mask`.
__device__ __forceinline__ void tc_commit_2cta(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;"
      ::"r"(bar), "h"(cta_mask) : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp receives lane
// (lane field of taddr) + t, columns [col, col+16).
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Same, 32 consecutive columns.
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Same wait, naming the registers an earlier tcgen05.ld fills: uses of r[] cannot be scheduled
// above it, which matters when other work is placed between the load and its wait.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]),
                 "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

// ------------------------------------------------------------------------------------
// Descriptors
// ------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major operand, rows of `swizzle_bytes` bytes
// (128 / 64 / 32, or 0 for the un-swizzled 8x16-byte core-matrix layout).
//   bits  0-13 start address >> 4        bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4   bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 swizzle mode (0 none, 2 = 128B, 4 = 64B, 6 = 32B)
// The stride byte offset is the distance between consecutive groups of 8 rows.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t stride_bytes,
                                                   uint32_t swizzle_bytes) {
  uint64_t mode = swizzle_bytes == 128 ? 2 : swizzle_bytes == 64 ? 4 : swizzle_bytes == 32 ? 6 : 0;
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;  // leading byte offset: unused by these layouts
  d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= mode << 61;
  return d;
}

// Instruction descriptor for kind::i8, signed 8-bit A and B (both K-major), int32 D.
//   bit 2 sparse flag; bits 4-5 D format (2 = s32); bits 7-9 A format (1 = s8);
//   bits 10-12 B format; bits 17-22 N>>3; bits 24-28 M>>4.
__host__ __device__ constexpr uint32_t make_idesc_i8(uint32_t m, uint32_t n, bool sparse) {
  return (sparse ? (1u << 2) : 0u) | (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// ------------------------------------------------------------------------------------
// Epilogue arithmetic shared by the dense and sparse GEMMs
// ------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_erf(float v) {
  return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
}

template <typename T>
__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i);

__device__ __forceinline__ float load_scalar(const void* p, int dtype, int64_t i) {
  if (dtype == HY3D_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == HY3D_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ uint32_t pack2(float a, float b, int out_dtype) {
  if (out_dtype == HY3D_BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}


// Host side: launch attribute that lets a kernel start before its stream predecessor ends
// (HY3D_PDL=0 in the environment turns it off).
inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("HY3D_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}
inline cudaLaunchAttribute pdl_attribute() {
  cudaLaunchAttribute a = {};
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  return a;
}

}  // namespace hy3d
