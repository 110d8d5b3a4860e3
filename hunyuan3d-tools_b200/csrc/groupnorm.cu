// GroupNorm (+ optional SiLU) over channels-last activations, for the UNet that surrounds the
// INT8 linear layers: x is (B, H*W, C) with C contiguous (torch's channels_last NCHW tensor),
// groups are runs of C / groups adjacent channels, statistics run over H*W x (C / groups)
// elements per (sample, group).  torch's own GroupNorm kernel takes NCHW only, so a model whose
// convolutions run NHWC pays two layout copies around every normalisation; this pair of
// kernels reads the NHWC tensor twice (the second time mostly from L2) and writes it once.
//
//   pass 1  groupnorm_stats_kernel   per (sample, row chunk): per-channel sum and sum of squares
//                                    in fp32 registers, folded into per-group partials
//                                    (fixed order, no atomics: results do not depend on timing)
//   pass 2  groupnorm_apply_kernel   mean / rstd per group from the partials, then
//                                    y = x * (rstd * gamma[c]) + (beta[c] - mean * rstd * gamma[c]),
//                                    rounded to the activation type; with silu != 0 the rounded
//                                    value goes through v / (1 + exp(-v)) and is rounded again
//                                    (the two roundings of GroupNorm followed by SiLU as
//                                    separate ops)
// Nothing here has a counterpart in the reference, whose UNet is stock PyTorch / diffusers.
#include "common.cuh"

namespace hy3d {
int device_sm_count();
namespace gnorm {
namespace {

constexpr int kMaxThreads = 320;

template <bool kBf16>
__device__ __forceinline__ void unpack8f(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (kBf16) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    } else {
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}

// x + add[b, c], rounded to the activation type as a separate broadcast add would have stored it.
template <bool kBf16>
__device__ __forceinline__ void add_round8(float (&f)[8], const float (&a)[8]) {
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    const uint32_t p = pack2(f[j] + a[j], f[j + 1] + a[j + 1], kBf16 ? HY3D_BF16 : HY3D_F16);
    if (kBf16) {
      f[j] = __uint_as_float(p << 16);
      f[j + 1] = __uint_as_float(p & 0xFFFF0000u);
    } else {
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&p));
      f[j] = t.x;
      f[j + 1] = t.y;
    }
  }
}

// Threads are laid out as (row lane ty, vector column tx): tx = tid % (C/8) owns 8 adjacent
// channels, ty = tid / (C/8) walks rows ty, ty + k, ...  blockDim.x = (C/8) * k.
//
// partial layout: [B][chunks][groups][2] floats (sum, sum of squares).
template <bool kBf16, bool kAdd>
__global__ void __launch_bounds__(kMaxThreads, kAdd ? 4 : 0)
groupnorm_stats_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ add, int64_t HW, int C,
                       int groups, int rows_per_chunk, float* __restrict__ partial) {
  extern __shared__ float s_acc[];          // [k][2][C]: per row lane, per-channel sum / sum of squares
  pdl_launch_dependents();
  const int vec_cols = C >> 3;
  const int k = blockDim.x / vec_cols;
  const int tx = threadIdx.x % vec_cols, ty = threadIdx.x / vec_cols;
  const int chunk = blockIdx.x, b = blockIdx.y, chunks = gridDim.x;
  const int64_t r0 = static_cast<int64_t>(chunk) * rows_per_chunk;
  const int64_t r1 = r0 + rows_per_chunk < HW ? r0 + rows_per_chunk : HW;
  pdl_wait();
  float s[8], q[8], av[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { s[j] = 0.0f; q[j] = 0.0f; av[j] = 0.0f; }
  if (kAdd) unpack8f<kBf16>(__ldg(reinterpret_cast<const uint4*>(add + static_cast<int64_t>(b) * C) + tx), av);
  const uint4* base = reinterpret_cast<const uint4*>(x + (static_cast<int64_t>(b) * HW) * C) + tx;
  int64_t r = r0 + ty;
  // four rows in flight per thread
  for (; r + 3 * k < r1; r += 4 * k) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldg(base + (r + u * k) * vec_cols);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float f[8];
      unpack8f<kBf16>(v[u], f);
      if (kAdd) add_round8<kBf16>(f, av);
#pragma unroll
      for (int j = 0; j < 8; ++j) { s[j] += f[j]; q[j] = fmaf(f[j], f[j], q[j]); }
    }
  }
  for (; r < r1; r += k) {
    float f[8];
    unpack8f<kBf16>(__ldg(base + r * vec_cols), f);
    if (kAdd) add_round8<kBf16>(f, av);
#pragma unroll
    for (int j = 0; j < 8; ++j) { s[j] += f[j]; q[j] = fmaf(f[j], f[j], q[j]); }
  }
  // Every row lane parks its sums in its own slice; channel c then adds the k slices in order.
  float* mine = s_acc + static_cast<size_t>(ty) * 2 * C;
#pragma unroll
  for (int j = 0; j < 8; ++j) { mine[8 * tx + j] = s[j]; mine[C + 8 * tx + j] = q[j]; }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * C; c += blockDim.x) {
    float a = s_acc[c];
    for (int lane = 1; lane < k; ++lane) a += s_acc[static_cast<size_t>(lane) * 2 * C + c];
    s_acc[c] = a;
  }
  __syncthreads();
  const int cpg = C / groups;
  float* out = partial + ((static_cast<int64_t>(b) * chunks + chunk) * groups) * 2;
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    float a = 0.0f, bq = 0.0f;
    for (int c = g * cpg; c < (g + 1) * cpg; ++c) { a += s_acc[c]; bq += s_acc[C + c]; }
    out[2 * g] = a;
    out[2 * g + 1] = bq;
  }
}

template <bool kBf16, bool kAdd>
__global__ void __launch_bounds__(kMaxThreads, 4)   // four resident blocks: the grid is sized as one such wave
groupnorm_apply_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ add, int64_t HW, int C, int groups,
                       int rows_per_chunk, int stat_chunks, const float* __restrict__ partial,
                       const void* __restrict__ gamma, const void* __restrict__ beta, int gb_dtype,
                       float eps, int silu, uint16_t* __restrict__ y) {
  extern __shared__ float s_ab[];           // [C] scale, [C] shift, then the partial-sum scratch
  pdl_launch_dependents();
  const int vec_cols = C >> 3;
  const int k = blockDim.x / vec_cols;
  const int tx = threadIdx.x % vec_cols, ty = threadIdx.x / vec_cols;
  const int chunk = blockIdx.x, b = blockIdx.y;
  const int cpg = C / groups;
  pdl_wait();
  const float inv_n = 1.0f / (static_cast<float>(HW) * static_cast<float>(cpg));
  // Partials -> per-group totals: `parts` threads share a group's chunks (a few independent
  // loads each instead of one thread walking all of them), then fold in fixed order.
  float* s_red = s_ab + 2 * C;               // [parts][groups][2]
  const int parts = static_cast<int>(blockDim.x) / groups > 0 ? static_cast<int>(blockDim.x) / groups : 1;
  for (int idx = threadIdx.x; idx < parts * groups; idx += blockDim.x) {
    const int g = idx % groups, part = idx / groups;
    const float* p = partial + (static_cast<int64_t>(b) * stat_chunks * groups + g) * 2;
    float a = 0.0f, q = 0.0f;
    for (int ch = part; ch < stat_chunks; ch += parts) {
      a += p[static_cast<int64_t>(ch) * 2 * groups];
      q += p[static_cast<int64_t>(ch) * 2 * groups + 1];
    }
    s_red[2 * idx] = a;
    s_red[2 * idx + 1] = q;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const int g = c / cpg;
    float a = 0.0f, q = 0.0f;
    for (int part = 0; part < parts; ++part) {
      a += s_red[2 * (part * groups + g)];
      q += s_red[2 * (part * groups + g) + 1];
    }
    const float mean = a * inv_n;
    const float var = fmaxf(fmaf(-mean, mean, q * inv_n), 0.0f);
    const float rstd = rsqrtf(var + eps);
    const float ga = gamma ? load_scalar(gamma, gb_dtype, c) : 1.0f;
    const float be = beta ? load_scalar(beta, gb_dtype, c) : 0.0f;
    s_ab[c] = rstd * ga;
    s_ab[C + c] = fmaf(-mean, rstd * ga, be);
  }
  __syncthreads();
  float sc[8], sh[8], av[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { sc[j] = s_ab[8 * tx + j]; sh[j] = s_ab[C + 8 * tx + j]; av[j] = 0.0f; }
  if (kAdd) unpack8f<kBf16>(__ldg(reinterpret_cast<const uint4*>(add + static_cast<int64_t>(b) * C) + tx), av);
  const int64_t r0 = static_cast<int64_t>(chunk) * rows_per_chunk;
  const int64_t r1 = r0 + rows_per_chunk < HW ? r0 + rows_per_chunk : HW;
  const int64_t sample = (static_cast<int64_t>(b) * HW) * C;
  const uint4* src = reinterpret_cast<const uint4*>(x + sample) + tx;
  uint4* dst = reinterpret_cast<uint4*>(y + sample) + tx;
  auto transform = [&](const uint4& v) {
    float f[8];
    unpack8f<kBf16>(v, f);
    if (kAdd) add_round8<kBf16>(f, av);
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      float y0 = fmaf(f[j], sc[j], sh[j]), y1 = fmaf(f[j + 1], sc[j + 1], sh[j + 1]);
      uint32_t packed = pack2(y0, y1, kBf16 ? HY3D_BF16 : HY3D_F16);
      if (silu) {
        if (kBf16) {
          y0 = __uint_as_float(packed << 16);
          y1 = __uint_as_float(packed & 0xFFFF0000u);
        } else {
          const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&packed));
          y0 = t.x; y1 = t.y;
        }
        // fast exp / divide: their error is far below half a unit of the 16-bit result
        y0 = __fdividef(y0, 1.0f + __expf(-y0));
        y1 = __fdividef(y1, 1.0f + __expf(-y1));
        packed = pack2(y0, y1, kBf16 ? HY3D_BF16 : HY3D_F16);
      }
      w[j >> 1] = packed;
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  };
  int64_t r = r0 + ty;
  for (; r + k < r1; r += 2 * k) {              // two rows in flight per thread
    const uint4 v0 = __ldg(src + r * vec_cols), v1 = __ldg(src + (r + k) * vec_cols);
    dst[r * vec_cols] = transform(v0);
    dst[(r + k) * vec_cols] = transform(v1);
  }
  for (; r < r1; r += k) dst[r * vec_cols] = transform(__ldg(src + r * vec_cols));
}

}  // namespace

// Rows per chunk so that B * chunks blocks fill the GPU a few times over; the statistics pass
// and the apply pass may use different chunkings (the apply pass is told the statistics' count).
int chunks_for(int64_t B, int64_t HW) {
  // One full wave: four 320-thread blocks are resident per SM (48 registers per thread), and a
  // grid that spills a few blocks into a second wave takes twice as long.
  const int sms = device_sm_count() > 0 ? device_sm_count() : 148;
  int64_t want = (static_cast<int64_t>(sms) * 4) / B;   // blocks per sample, rounded down
  if (want < 1) want = 1;
  if (want > 64) want = 64;
  int64_t rows = (HW + want - 1) / want;
  if (rows < 8) rows = 8;
  return static_cast<int>((HW + rows - 1) / rows);
}

int64_t workspace_floats(int64_t B, int64_t HW, int groups) {
  return B * chunks_for(B, HW) * groups * 2;
}

int groupnorm_nhwc(const void* x, const void* add, int x_dtype, int64_t B, int64_t HW, int64_t C, int groups,
                   const void* gamma, const void* beta, int gb_dtype, float eps, int silu,
                   void* y, float* workspace, cudaStream_t stream) {
  if (x_dtype != HY3D_F16 && x_dtype != HY3D_BF16) return HY3D_ERR_ARG;
  if ((gamma || beta) && (gb_dtype < HY3D_F16 || gb_dtype > HY3D_F32)) return HY3D_ERR_ARG;
  if (B < 0 || HW <= 0 || C <= 0 || groups <= 0 || (C & 7) || C % groups) return HY3D_ERR_SHAPE;
  if (C > 8 * kMaxThreads || B > 65535 || HW > (1ll << 31)) return HY3D_ERR_SHAPE;
  if (B == 0) return HY3D_OK;
  if (!x || !y || !workspace) return HY3D_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(add)) & 15)
    return HY3D_ERR_SHAPE;
  const int Ci = static_cast<int>(C);
  const int vec_cols = Ci >> 3;
  const int k = kMaxThreads / vec_cols > 0 ? kMaxThreads / vec_cols : 1;
  const int threads = vec_cols * k;
  const int chunks = chunks_for(B, HW);
  const int rows_per_chunk = static_cast<int>((HW + chunks - 1) / chunks);
  const int parts = threads / groups > 0 ? threads / groups : 1;
  const size_t smem = (static_cast<size_t>(2 * Ci) + static_cast<size_t>(parts) * groups * 2) * sizeof(float);  // apply
  const size_t smem_stats = static_cast<size_t>(k) * 2 * Ci * sizeof(float);  // stats: one slice per row lane
  const bool bf16 = x_dtype == HY3D_BF16;
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  uint16_t* yp = static_cast<uint16_t*>(y);
  const uint16_t* ap = static_cast<const uint16_t*>(add);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(chunks), static_cast<unsigned>(B));
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0] = pdl_attribute();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t err;
  cfg.dynamicSmemBytes = smem_stats;
#define HY3D_GN_STATS(BF, AD) \
  err = cudaLaunchKernelEx(&cfg, groupnorm_stats_kernel<BF, AD>, xp, ap, HW, Ci, groups, rows_per_chunk, workspace)
  if (bf16) { if (ap) HY3D_GN_STATS(true, true); else HY3D_GN_STATS(true, false); }
  else { if (ap) HY3D_GN_STATS(false, true); else HY3D_GN_STATS(false, false); }
#undef HY3D_GN_STATS
  if (err != cudaSuccess) { cudaGetLastError(); return HY3D_ERR_CUDA; }
  const float* ws = workspace;
  cfg.dynamicSmemBytes = smem;
#define HY3D_GN_APPLY(BF, AD)                                                                       \
  err = cudaLaunchKernelEx(&cfg, groupnorm_apply_kernel<BF, AD>, xp, ap, HW, Ci, groups, rows_per_chunk, \
                           chunks, ws, gamma, beta, gb_dtype, eps, silu, yp)
  if (bf16) { if (ap) HY3D_GN_APPLY(true, true); else HY3D_GN_APPLY(true, false); }
  else { if (ap) HY3D_GN_APPLY(false, true); else HY3D_GN_APPLY(false, false); }
#undef HY3D_GN_APPLY
  if (err != cudaSuccess) { cudaGetLastError(); return HY3D_ERR_CUDA; }
  return HY3D_OK;
}

}  // namespace gnorm
}  // namespace hy3d
