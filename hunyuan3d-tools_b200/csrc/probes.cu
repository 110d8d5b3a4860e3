// Measurement hooks: the denominators the benchmark reports its kernels against, measured on
// the GPU at hand with the same instructions the kernels use.  None of this is on the product
// path, and nothing here has a counterpart in the reference.
//   hy3d_probe_mma_i8   resident-operand tcgen05.mma kind::i8 issue loop on every SM: the
//                       practical INT8 tensor peak (dense or 2:4 sparse) under the power cap
//   hy3d_probe_hbm      write-only / read-only / copy streams over a caller-provided buffer
//   hy3d_probe_tmem_ld  tensor-memory -> register drain rate (tcgen05.ld 32x32b.x16) with a
//                       chosen number of warps and loads in flight per warp
#include "common.cuh"

namespace hy3d {
int ensure_max_smem(const void* kernel, int bytes);
int device_sm_count();

namespace probe {
namespace {

constexpr int kProbeSmem = 96 * 1024;

// One CTA per SM.  Operands (A 128 x 128 B, B n x 128 B, both 128-byte swizzled; for the
// sparse form A is the compressed operand and its metadata sits in tensor memory) stay in
// shared memory; one thread issues groups of four MMAs (one 128-deep K block) and commits each
// group to one of two barriers, waiting for the group issued two earlier -- the cadence of a
// two-stage pipeline, without any loads.
template <bool kSparse>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int n, int groups) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bars[3];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 3; ++i) mbar_init(smem_u32(&bars[i]), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < kProbeSmem / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem)[i] = 0x01010101u;
  if (warp == 0) {
    tmem_alloc_1cta(smem_u32(&tmem_base_s), 512);
    tmem_relinquish_1cta();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  if (warp == 1 && lane == 0) {
    const uint32_t idesc = make_idesc_i8(128, static_cast<uint32_t>(n), kSparse);
    const uint64_t desc = make_smem_desc(0, 1024, 128);
    const uint32_t sa = smem_u32(smem);
    const uint64_t da = desc | static_cast<uint64_t>((sa & 0x3FFFFu) >> 4);
    const uint64_t db = desc | static_cast<uint64_t>(((sa + 16384) & 0x3FFFFu) >> 4);
    const uint32_t e_tmem = tmem_base + 256;   // metadata columns (contents irrelevant to the rate)
    uint32_t phase[2] = {0, 0};
    bool ok = true;
    for (int g = 0; ok && g < groups; ++g) {
      const int b = g & 1;
      if (g >= 2) {
        ok = mbar_wait<true>(smem_u32(&bars[b]), phase[b], &abort_flag, kDevTimeoutFull);
        phase[b] ^= 1;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (kSparse) mma_sp_i8_1cta(tmem_base, da + 2 * k, db + 4 * (k & 1), e_tmem + 2 * k, idesc, 1u);
        else mma_i8_1cta(tmem_base, da + 2 * k, db + 2 * k, idesc, 1u);
      }
      tc_commit_1cta(smem_u32(&bars[b]));
    }
    if (ok) {
      tc_commit_1cta(smem_u32(&bars[2]));   // covers everything issued before it
      mbar_wait<true>(smem_u32(&bars[2]), 0, &abort_flag, kDevTimeoutFull);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc_1cta(tmem_base, 512);
  }
}

// mode 0: write-only, 1: read-only (a checksum keeps the loads alive), 2: copy a -> b.
__global__ void __launch_bounds__(512) hbm_stream_kernel(uint4* __restrict__ a, uint4* __restrict__ b,
                                                         int64_t nvec, int mode, uint32_t* sink) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  uint32_t acc = 0;
  if (mode == 0) {
    const uint4 v = make_uint4(1u, 2u, 3u, static_cast<uint32_t>(i));
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      __stcs(a + i, v); __stcs(a + i + stride, v); __stcs(a + i + 2 * stride, v); __stcs(a + i + 3 * stride, v);
    }
    for (; i < nvec; i += stride) __stcs(a + i, v);
  } else if (mode == 1) {
    for (; i + 7 * stride < nvec; i += 8 * stride) {   // eight 16-byte loads in flight per thread
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __ldcs(a + i + j * stride);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc ^= v[j].x ^ v[j].y ^ v[j].z ^ v[j].w;
    }
    for (; i < nvec; i += stride) { const uint4 v = __ldcs(a + i); acc ^= v.x ^ v.y ^ v.z ^ v.w; }
    if (acc == 0x9E3779B9u) *sink = acc;   // practically never true; defeats dead-code elimination
  } else {
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      const uint4 v0 = __ldcs(a + i), v1 = __ldcs(a + i + stride), v2 = __ldcs(a + i + 2 * stride),
                  v3 = __ldcs(a + i + 3 * stride);
      __stcs(b + i, v0); __stcs(b + i + stride, v1); __stcs(b + i + 2 * stride, v2); __stcs(b + i + 3 * stride, v3);
    }
    for (; i < nvec; i += stride) __stcs(b + i, __ldcs(a + i));
  }
}

__device__ uint32_t g_probe_sink;

// One CTA per SM, `blockDim.x / 32` warps.  Every warp reads its lane quarter of tensor memory
// `iters` times: kDepth loads of 16 columns are issued back to back, then one wait.
template <int kDepth>
__global__ void __launch_bounds__(512, 1) tmem_drain_kernel(int iters, uint32_t* sink) {
  __shared__ uint32_t tmem_base_s;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    tmem_alloc_1cta(smem_u32(&tmem_base_s), 512);
    tmem_relinquish_1cta();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t t_row = tmem_base_s + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  uint32_t acc = 0;
  uint32_t col = static_cast<uint32_t>(warp >> 2) * 64u;
  for (int i = 0; i < iters; ++i) {
    uint32_t r[kDepth][16];
#pragma unroll
    for (int d = 0; d < kDepth; ++d) tmem_ld_x16(t_row + ((col + 16u * d) & 511u), r[d]);
#pragma unroll
    for (int d = 0; d < kDepth; ++d) tmem_ld_wait_for(r[d]);
#pragma unroll
    for (int d = 0; d < kDepth; ++d) acc ^= r[d][0] ^ r[d][7] ^ r[d][15];
    col = (col + 16u * kDepth) & 511u;
  }
  if (acc == 0x9E3779B9u) *sink = acc;
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc_1cta(tmem_base_s, 512);
  }
}

}  // namespace
}  // namespace probe
}  // namespace hy3d

extern "C" {

int hy3d_probe_mma_i8(int n, int groups, int sparse, int64_t* ops_out, void* stream) {
  using namespace hy3d;
  if (n < 16 || n > 256 || (n & 15) || groups < 1 || groups > (1 << 24)) return HY3D_ERR_SHAPE;
  const int sms = device_sm_count();
  if (sms <= 0) return HY3D_ERR_CUDA;
  const void* fn = sparse ? reinterpret_cast<const void*>(probe::mma_rate_kernel<true>)
                          : reinterpret_cast<const void*>(probe::mma_rate_kernel<false>);
  const int rc = ensure_max_smem(fn, probe::kProbeSmem);
  if (rc != HY3D_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (sparse) probe::mma_rate_kernel<true><<<sms, 128, probe::kProbeSmem, s>>>(n, groups);
  else probe::mma_rate_kernel<false><<<sms, 128, probe::kProbeSmem, s>>>(n, groups);
  // Dense-equivalent operations of the launch: a sparse instruction covers 64 logical K.
  if (ops_out)
    *ops_out = static_cast<int64_t>(sms) * groups * 4 * 2 * 128 * n * (sparse ? 64 : 32);
  return cudaGetLastError() == cudaSuccess ? HY3D_OK : HY3D_ERR_CUDA;
}

int hy3d_probe_tmem_ld(int warps, int depth, int iters, int64_t* bytes_out, void* stream) {
  using namespace hy3d;
  if (warps < 4 || warps > 16 || (warps & 3) || iters < 1 || iters > (1 << 24)) return HY3D_ERR_ARG;
  if (depth != 1 && depth != 2 && depth != 4) return HY3D_ERR_ARG;
  const int sms = device_sm_count();
  if (sms <= 0) return HY3D_ERR_CUDA;
  uint32_t* sink = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&sink), probe::g_probe_sink) != cudaSuccess)
    return HY3D_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (depth == 1) probe::tmem_drain_kernel<1><<<sms, warps * 32, 0, s>>>(iters, sink);
  else if (depth == 2) probe::tmem_drain_kernel<2><<<sms, warps * 32, 0, s>>>(iters, sink);
  else probe::tmem_drain_kernel<4><<<sms, warps * 32, 0, s>>>(iters, sink);
  if (bytes_out) *bytes_out = static_cast<int64_t>(sms) * warps * iters * depth * 2048;
  return cudaGetLastError() == cudaSuccess ? HY3D_OK : HY3D_ERR_CUDA;
}

int hy3d_probe_hbm(int mode, void* a, void* b, int64_t bytes, void* stream) {
  using namespace hy3d;
  if (mode < 0 || mode > 2 || !a || (mode == 2 && !b) || bytes < 16 || (bytes & 15)) return HY3D_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) return HY3D_ERR_SHAPE;
  const int sms = device_sm_count();
  if (sms <= 0) return HY3D_ERR_CUDA;
  uint32_t* sink = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&sink), probe::g_probe_sink) != cudaSuccess)
    return HY3D_ERR_CUDA;
  probe::hbm_stream_kernel<<<sms * 4, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(a), static_cast<uint4*>(b), bytes / 16, mode, sink);
  return cudaGetLastError() == cudaSuccess ? HY3D_OK : HY3D_ERR_CUDA;
}

}  // extern "C"
