// Per-token absmax activation quantiser and the stand-alone dequant+bias epilogue kernel.
//
// Quantiser arithmetic (bit-exact contract, checked against the CPU oracle):
//     amax  = max_k |x[m,k]|                       (fp32)
//     scale = max(amax, 1e-8f) / 127.0f            (IEEE division)
//     q     = clamp(rint(x / scale), -128, 127)    (IEEE division, round-half-even)
// The row is read ONCE with 16-byte loads and kept in registers between the absmax
// reduction and the rounding pass, so the kernel moves 2*K + K + 4/M bytes per row.
// 16-bit activations sit on a coarse grid, so quotients within rounding error of k + 0.5 are
// common (about 0.2 % of the elements of a Gaussian bf16 row) and their codes depend on the
// last bit of the IEEE quotient.  The quotient is therefore refined without a division
// instruction: q0 = x * rcp(scale) with the correctly rounded reciprocal, then one residual
// correction r = fma(-q0, scale, x); q = fma(r, rcp, q0).  A device-side enumeration of every
// pair of 16-bit patterns (amax, x) with |x| <= amax -- 1.0e9 pairs for fp16, 1.07e9 for bf16,
// i.e. every input this kernel can see -- found rint(q) == rint(__fdiv_rn(x, scale)) for all of
// them (without the correction 16732 / 7424 pairs differ).
#include "common.cuh"

namespace hy3d {
namespace quant {
namespace {

constexpr int kQuantThreads = 256;

template <bool kBf16>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (kBf16) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    } else {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}

// Folds the eight 16-bit values of a 16-byte vector into a running packed |x| maximum
// (two lanes per register), without widening them first.
template <bool kBf16>
__device__ __forceinline__ void absmax8(const uint4& v, uint32_t& acc) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (kBf16) {
      const __nv_bfloat162 m = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&acc),
                                       __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[i])));
      acc = *reinterpret_cast<const uint32_t*>(&m);
    } else {
      const __half2 m = __hmax2(*reinterpret_cast<const __half2*>(&acc),
                                __habs2(*reinterpret_cast<const __half2*>(&w[i])));
      acc = *reinterpret_cast<const uint32_t*>(&m);
    }
  }
}
template <bool kBf16>
__device__ __forceinline__ float absmax_to_float(uint32_t acc) {
  if (kBf16) {
    return fmaxf(__uint_as_float(acc << 16), __uint_as_float(acc & 0xFFFF0000u));
  }
  const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&acc));
  return fmaxf(t.x, t.y);
}

// Quantises eight values to eight int8 codes (two words).  Float <-> int conversion
// instructions run at a fraction of the FMA rate on this architecture, so the final rounding
// uses the 1.5 * 2^23 trick: adding that constant rounds |t| < 2^22 to the nearest integer
// (ties to even, the FPU's own rounding) and leaves the two's-complement code in the low
// mantissa byte, which a byte permute then gathers.  t is the refined quotient of the file
// header, whose rounding equals that of the IEEE quotient for every 16-bit input.
// No clamp is needed: scale = max|x| / 127 bounds |x / scale| by 127 (+ one rounding).
__device__ __forceinline__ float refined_quotient(float x, float scale, float inv) {
  const float q0 = x * inv;
  return fmaf(fmaf(-q0, scale, x), inv, q0);
}
// The same for two values at once with the packed fp32x2 instructions of sm_100 (each half is
// an IEEE single-precision operation, so the results equal the scalar form bit for bit; the
// point is half as many issue slots).  Returns refined quotient + 1.5 * 2^23.
__device__ __forceinline__ float2 refined_quotient2_magic(float2 x, float scale, float inv) {
  const float2 inv2 = make_float2(inv, inv), nscale2 = make_float2(-scale, -scale);
  const float2 q0 = __fmul2_rn(x, inv2);
  const float2 r = __ffma2_rn(q0, nscale2, x);
  const float2 q = __ffma2_rn(r, inv2, q0);
  return __fadd2_rn(q, make_float2(12582912.0f, 12582912.0f));
}

__device__ __forceinline__ uint2 quant8(const float (&f)[8], float scale, float inv) {
  uint32_t b[8];
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    const float2 t = refined_quotient2_magic(make_float2(f[j], f[j + 1]), scale, inv);
    b[j] = __float_as_uint(t.x);
    b[j + 1] = __float_as_uint(t.y);
  }
  const uint32_t p01 = __byte_perm(b[0], b[1], 0x0040), p23 = __byte_perm(b[2], b[3], 0x0040);
  const uint32_t p45 = __byte_perm(b[4], b[5], 0x0040), p67 = __byte_perm(b[6], b[7], 0x0040);
  return make_uint2(__byte_perm(p01, p23, 0x5410), __byte_perm(p45, p67, 0x5410));
}

// G threads cooperate on one row (G a power of two, 1..256); each holds up to kMaxV
// 16-byte vectors.  A block of 256 threads covers 256/G rows.
template <bool kBf16, int kMaxV>
__global__ void __launch_bounds__(kQuantThreads, kMaxV <= 5 ? 4 : 3)
quantize_rows_kernel(const uint16_t* __restrict__ x, int64_t ldx, int8_t* __restrict__ q,
                     float* __restrict__ scale_out, int64_t M, int K, int G) {
  __shared__ float s_part[kQuantThreads / 32];
  pdl_launch_dependents();
  pdl_wait();   // x comes from the previous kernel in the stream
  const int tid = threadIdx.x;
  const int rows_per_block = kQuantThreads / G;
  const int sub = tid % G;  // position within the row group
  const int64_t row = static_cast<int64_t>(blockIdx.x) * rows_per_block + tid / G;
  const bool row_ok = row < M;
  const int nvec = K >> 3;

  uint4 v[kMaxV];
  uint32_t amax2 = 0;
  const uint4* src = reinterpret_cast<const uint4*>(x + (row_ok ? row : 0) * ldx);
#pragma unroll
  for (int i = 0; i < kMaxV; ++i) {
    const int c = sub + i * G;
    if (row_ok && c < nvec) {
      v[i] = __ldcs(src + c);
    } else {
      v[i] = make_uint4(0, 0, 0, 0);
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxV; ++i) absmax8<kBf16>(v[i], amax2);
  float amax = absmax_to_float<kBf16>(amax2);
  // Reduce over the G threads of the row.
  const int w = G < 32 ? G : 32;
  for (int off = w >> 1; off > 0; off >>= 1)
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if (G > 32) {
    const int warp = tid >> 5;
    if ((tid & 31) == 0) s_part[warp] = amax;
    __syncthreads();
    const int warps_per_row = G >> 5;
    const int first = (warp / warps_per_row) * warps_per_row;
    amax = s_part[first];
    for (int i = 1; i < warps_per_row; ++i) amax = fmaxf(amax, s_part[first + i]);
  }
  const float scale = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
  const float inv = __frcp_rn(scale);
  if (row_ok && sub == 0) scale_out[row] = scale;

  uint2* dst = reinterpret_cast<uint2*>(q + (row_ok ? row : 0) * static_cast<int64_t>(K));
#pragma unroll
  for (int i = 0; i < kMaxV; ++i) {
    const int c = sub + i * G;
    if (row_ok && c < nvec) {
      float f[8];
      unpack8<kBf16>(v[i], f);
      dst[c] = quant8(f, scale, inv);
    }
  }
}

template <bool kBf16>
int launch_quantize(const void* x, int64_t M, int64_t K, int64_t ldx, int8_t* q, float* scale,
                    cudaStream_t stream) {
  const int nvec = static_cast<int>(K >> 3);
  // Choose the power-of-two group size G and vectors-per-thread V (<= 8) that cover the row
  // with the fewest idle vector slots; among equals prefer V near 4 (enough loads in flight
  // per thread without starving the block of rows).
  int G = 0, maxv = 0, best = 1 << 30;
  for (int g = 1; g <= kQuantThreads; g <<= 1) {
    const int v = (nvec + g - 1) / g;
    if (v > 8) continue;
    const int score = (g * v - nvec) * 1000 / nvec * 16 + (v > 4 ? v - 4 : 4 - v);
    if (score < best) { best = score; G = g; maxv = v; }
  }
  if (G == 0) return HY3D_ERR_SHAPE;
  const int rows_per_block = kQuantThreads / G;
  const int64_t blocks = (M + rows_per_block - 1) / rows_per_block;
  if (blocks > 0x7FFFFFFF) return HY3D_ERR_SHAPE;
  const uint16_t* xp = reinterpret_cast<const uint16_t*>(x);
  dim3 grid(static_cast<unsigned>(blocks));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kQuantThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1] = {pdl_attribute()};
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t err = cudaSuccess;
  const int Ki = static_cast<int>(K);
#define HY3D_LAUNCH_Q(V) \
  err = cudaLaunchKernelEx(&cfg, quantize_rows_kernel<kBf16, V>, xp, ldx, q, scale, M, Ki, G)
  switch (maxv) {
    case 1: HY3D_LAUNCH_Q(1); break;
    case 2: HY3D_LAUNCH_Q(2); break;
    case 3: HY3D_LAUNCH_Q(3); break;
    case 4: HY3D_LAUNCH_Q(4); break;
    case 5: HY3D_LAUNCH_Q(5); break;
    case 6: HY3D_LAUNCH_Q(6); break;
    case 7: HY3D_LAUNCH_Q(7); break;
    default: HY3D_LAUNCH_Q(8); break;
  }
#undef HY3D_LAUNCH_Q
  if (err != cudaSuccess) {
    cudaGetLastError();
    return HY3D_ERR_CUDA;
  }
  return HY3D_OK;
}

// LayerNorm fused with the per-token quantiser: the row is normalised in registers, rounded to
// the 16-bit activation type exactly as a stand-alone LayerNorm would store it, and those
// rounded values are quantised with the arithmetic above -- so the codes and scales equal
// quantize_rows(LayerNorm(x)) bit for bit while the normalised activations never go to memory
// (x is read once: 2*K bytes in, K + 4 bytes out per row, instead of 2K + 2K for the LayerNorm
// and 2K + K for the quantiser).  Arithmetic, all fp32, fixed reduction order:
//     mean = sum(x) / K;  var = sum((x - mean)^2) / K;  rstd = 1 / sqrt(var + eps)  (IEEE)
//     y    = round16( fma((x - mean) * rstd, gamma, beta) )
// G <= 32 lanes share a row (shuffle reductions); gamma / beta are staged once per block in
// shared memory as fp32 and the block walks rows with a grid-stride loop.
template <bool kBf16, int kMaxV>
__global__ void __launch_bounds__(kQuantThreads, kMaxV <= 4 ? 3 : 2)
layernorm_quantize_kernel(const uint16_t* __restrict__ x, int64_t ldx, const void* __restrict__ gamma,
                          const void* __restrict__ beta, int gb_dtype, float eps,
                          int8_t* __restrict__ q, float* __restrict__ scale_out,
                          uint16_t* __restrict__ y_out, int64_t M, int K, int G) {
  extern __shared__ float s_gb[];            // gamma and beta as fp32, 2 * K floats in planes
  pdl_launch_dependents();
  // Four planes of K/8 float4 each: [gamma 0-3 | gamma 4-7 | beta 0-3 | beta 4-7] of every
  // 8-element vector, so that the 16-byte loads of neighbouring lanes (neighbouring vectors)
  // are contiguous and conflict-free.
  const int plane = (K >> 3) * 4;
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const int at = ((k >> 2) & 1) * plane + (k >> 3) * 4 + (k & 3);
    s_gb[at] = gamma ? load_scalar(gamma, gb_dtype, k) : 1.0f;
    s_gb[2 * plane + at] = beta ? load_scalar(beta, gb_dtype, k) : 0.0f;
  }
  pdl_wait();   // x comes from the previous kernel in the stream; gamma / beta are parameters
  __syncthreads();
  const int tid = threadIdx.x;
  const int rows_per_block = kQuantThreads / G;
  const int sub = tid % G;
  const int nvec = K >> 3;
  const float inv_k = 1.0f / static_cast<float>(K);
  // The next row's vectors are requested before the current row is worked on, so that every
  // warp keeps loads in flight through its reductions.
  const int64_t row_step = static_cast<int64_t>(gridDim.x) * rows_per_block;
  uint4 vn[kMaxV];
  auto fetch = [&](int64_t r0) {
    const int64_t r = r0 + tid / G;
    const uint4* src = reinterpret_cast<const uint4*>(x + (r < M ? r : 0) * ldx);
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int c = sub + i * G;
      vn[i] = (r < M && c < nvec) ? __ldcs(src + c) : make_uint4(0, 0, 0, 0);
    }
  };
  fetch(static_cast<int64_t>(blockIdx.x) * rows_per_block);
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_block; row0 < M; row0 += row_step) {
    const int64_t row = row0 + tid / G;
    const bool row_ok = row < M;
    // The row lives in registers as pairs; every step below is a packed fp32x2 instruction
    // (two IEEE single-precision operations per issue slot).
    float2 f[kMaxV][4];
    float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      float t[8];
      unpack8<kBf16>(vn[i], t);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f[i][j] = make_float2(t[2 * j], t[2 * j + 1]);
        sum2 = __fadd2_rn(sum2, f[i][j]);
      }
    }
    if (row0 + row_step < M) fetch(row0 + row_step);
    float sum = sum2.x + sum2.y;
    for (int off = G >> 1; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float mean = sum * inv_k;
    const float2 nmean2 = make_float2(-mean, -mean);
    float2 ss2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int c = sub + i * G;
      if (c < nvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          f[i][j] = __fadd2_rn(f[i][j], nmean2);          // centred from here on
          ss2 = __ffma2_rn(f[i][j], f[i][j], ss2);
        }
      }
    }
    float ss = ss2.x + ss2.y;
    for (int off = G >> 1; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float rstd = __frcp_rn(__fsqrt_rn(fmaf(ss, inv_k, eps)));
    const float2 rstd2 = make_float2(rstd, rstd);
    // normalise, round to the activation type, keep the rounded values for the quantiser
    uint32_t amax2 = 0;
    uint4 yv[kMaxV];
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int c = sub + i * G;
      yv[i] = make_uint4(0, 0, 0, 0);
      if (c < nvec) {
        const float4 g0 = *reinterpret_cast<const float4*>(s_gb + 4 * c);
        const float4 g1 = *reinterpret_cast<const float4*>(s_gb + plane + 4 * c);
        const float4 b0 = *reinterpret_cast<const float4*>(s_gb + 2 * plane + 4 * c);
        const float4 b1 = *reinterpret_cast<const float4*>(s_gb + 3 * plane + 4 * c);
        const float2 gg[4] = {make_float2(g0.x, g0.y), make_float2(g0.z, g0.w),
                              make_float2(g1.x, g1.y), make_float2(g1.z, g1.w)};
        const float2 bb[4] = {make_float2(b0.x, b0.y), make_float2(b0.z, b0.w),
                              make_float2(b1.x, b1.y), make_float2(b1.z, b1.w)};
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 y = __ffma2_rn(__fmul2_rn(f[i][j], rstd2), gg[j], bb[j]);
          if (kBf16) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(y.x, y.y);
            w[j] = *reinterpret_cast<const uint32_t*>(&h);
          } else {
            const __half2 h = __floats2half2_rn(y.x, y.y);
            w[j] = *reinterpret_cast<const uint32_t*>(&h);
          }
        }
        yv[i] = make_uint4(w[0], w[1], w[2], w[3]);
        absmax8<kBf16>(yv[i], amax2);
      }
    }
    float amax = absmax_to_float<kBf16>(amax2);
    for (int off = G >> 1; off > 0; off >>= 1)
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float scale = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
    const float inv = __frcp_rn(scale);
    if (row_ok && sub == 0) scale_out[row] = scale;
    uint2* dst = reinterpret_cast<uint2*>(q + (row_ok ? row : 0) * static_cast<int64_t>(K));
    uint4* ydst = y_out ? reinterpret_cast<uint4*>(y_out + (row_ok ? row : 0) * static_cast<int64_t>(K)) : nullptr;
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int c = sub + i * G;
      if (row_ok && c < nvec) {
        float fy[8];
        unpack8<kBf16>(yv[i], fy);
        dst[c] = quant8(fy, scale, inv);
        if (ydst) ydst[c] = yv[i];
      }
    }
  }
}

template <bool kBf16>
int launch_layernorm_quantize(const void* x, int64_t M, int64_t K, int64_t ldx, const void* gamma,
                              const void* beta, int gb_dtype, float eps, int8_t* q, float* scale,
                              void* y_out, cudaStream_t stream) {
  const int nvec = static_cast<int>(K >> 3);
  // lanes per row: the power of two (<= 32) that leaves at most 5 vectors per lane
  int G = 1;
  while (G < 32 && (nvec + G - 1) / G > 5) G <<= 1;
  const int maxv = (nvec + G - 1) / G;
  if (maxv > 8) return HY3D_ERR_SHAPE;
  const int rows_per_block = kQuantThreads / G;
  int64_t blocks = (M + rows_per_block - 1) / rows_per_block;
  const int64_t cap = 148 * 8;
  if (blocks > cap) blocks = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(kQuantThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(2 * K) * sizeof(float);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1] = {pdl_attribute()};
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const uint16_t* xp = reinterpret_cast<const uint16_t*>(x);
  uint16_t* yp = reinterpret_cast<uint16_t*>(y_out);
  const int Ki = static_cast<int>(K);
  cudaError_t err = cudaSuccess;
#define HY3D_LAUNCH_LNQ(V) \
  err = cudaLaunchKernelEx(&cfg, layernorm_quantize_kernel<kBf16, V>, xp, ldx, gamma, beta, gb_dtype, eps, \
                           q, scale, yp, M, Ki, G)
  if (maxv <= 2) HY3D_LAUNCH_LNQ(2);
  else if (maxv <= 4) HY3D_LAUNCH_LNQ(4);
  else if (maxv == 5) HY3D_LAUNCH_LNQ(5);
  else HY3D_LAUNCH_LNQ(8);
#undef HY3D_LAUNCH_LNQ
  if (err != cudaSuccess) {
    cudaGetLastError();
    return HY3D_ERR_CUDA;
  }
  return HY3D_OK;
}

// Enumeration behind the quantiser's exactness claim: block a takes the 16-bit pattern a as
// amax, its threads walk all 65536 patterns x with |x| <= amax and compare the code the
// quantiser's arithmetic produces with (int8) rint(x / scale) computed by IEEE division.
__device__ unsigned long long g_enum_counts[2];   // [0] pairs checked, [1] codes that differ

template <bool kBf16>
__global__ void __launch_bounds__(256) quotient_enum_kernel() {
  const uint32_t a_bits = blockIdx.x;
  const float amax = kBf16 ? __uint_as_float(a_bits << 16)
                           : __half2float(__ushort_as_half(static_cast<unsigned short>(a_bits)));
  if (!(amax == amax) || isinf(amax)) return;
  const float scale = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
  const float inv = __frcp_rn(scale);
  unsigned long long pairs = 0, bad = 0;
  // Two patterns per step, through the packed arithmetic the quantiser kernels run.
  for (uint32_t xb = 2 * threadIdx.x; xb < 65536u; xb += 2 * blockDim.x) {
    float x[2];
#pragma unroll
    for (int h = 0; h < 2; ++h)
      x[h] = kBf16 ? __uint_as_float((xb + h) << 16)
                   : __half2float(__ushort_as_half(static_cast<unsigned short>(xb + h)));
    const float2 t = refined_quotient2_magic(make_float2(x[0], x[1]), scale, inv);
    const uint32_t b[2] = {__float_as_uint(t.x), __float_as_uint(t.y)};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (!(fabsf(x[h]) <= amax)) continue;
      const int code = static_cast<int>(static_cast<signed char>(b[h] & 0xFFu));
      const int ref = static_cast<int>(rintf(__fdiv_rn(x[h], scale)));
      ++pairs;
      if (code != ref) ++bad;
    }
  }
  atomicAdd(&g_enum_counts[0], pairs);
  atomicAdd(&g_enum_counts[1], bad);
}

// out[m,n] = acc[m,n] * (act_scale[m] * w_scale[n]) + bias[n]; 8 columns per thread.
__global__ void __launch_bounds__(256)
dequant_bias_kernel(const int32_t* __restrict__ acc, const float* __restrict__ act_scale,
                    const void* __restrict__ w_scale, int ws_dtype, const void* __restrict__ bias,
                    int bias_dtype, void* __restrict__ out, int out_dtype, int64_t M, int64_t N) {
  const int64_t nchunk = N >> 3;
  const int64_t total = M * nchunk;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = i / nchunk;
    const int64_t n0 = (i - m * nchunk) << 3;
    const int4* src = reinterpret_cast<const int4*>(acc + m * N + n0);
    const int4 a0 = src[0], a1 = src[1];
    const int a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const float as = act_scale[m];
    float y[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = as * load_scalar(w_scale, ws_dtype, n0 + j);
      const float b = bias ? load_scalar(bias, bias_dtype, n0 + j) : 0.0f;
      y[j] = fmaf(static_cast<float>(a[j]), s, b);
    }
    uint4 o;
    o.x = pack2(y[0], y[1], out_dtype);
    o.y = pack2(y[2], y[3], out_dtype);
    o.z = pack2(y[4], y[5], out_dtype);
    o.w = pack2(y[6], y[7], out_dtype);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + m * N + n0) = o;
  }
}

}  // namespace

int quantize_rows(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* q,
                  float* scale, cudaStream_t stream) {
  if (x_dtype != HY3D_F16 && x_dtype != HY3D_BF16) return HY3D_ERR_ARG;
  if (M < 0 || K <= 0 || (K & 7) || K > 16384 || ldx < K || (ldx & 7)) return HY3D_ERR_SHAPE;
  if (M == 0) return HY3D_OK;
  if (!x || !q || !scale) return HY3D_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7))
    return HY3D_ERR_SHAPE;
  if (M == 0) return HY3D_OK;
  return x_dtype == HY3D_BF16 ? launch_quantize<true>(x, M, K, ldx, q, scale, stream)
                              : launch_quantize<false>(x, M, K, ldx, q, scale, stream);
}

int layernorm_quantize(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* gamma,
                       const void* beta, int gb_dtype, float eps, int8_t* q, float* scale, void* y_out,
                       cudaStream_t stream) {
  if (x_dtype != HY3D_F16 && x_dtype != HY3D_BF16) return HY3D_ERR_ARG;
  if ((gamma || beta) && (gb_dtype < HY3D_F16 || gb_dtype > HY3D_F32)) return HY3D_ERR_ARG;
  if (M < 0 || K <= 0 || (K & 7) || K > 2048 || ldx < K || (ldx & 7)) return HY3D_ERR_SHAPE;
  if (!(eps >= 0.0f)) return HY3D_ERR_ARG;
  if (M == 0) return HY3D_OK;
  if (!x || !q || !scale) return HY3D_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7) ||
      (reinterpret_cast<uintptr_t>(y_out) & 15))
    return HY3D_ERR_SHAPE;
  return x_dtype == HY3D_BF16
             ? launch_layernorm_quantize<true>(x, M, K, ldx, gamma, beta, gb_dtype, eps, q, scale, y_out, stream)
             : launch_layernorm_quantize<false>(x, M, K, ldx, gamma, beta, gb_dtype, eps, q, scale, y_out, stream);
}

int quantizer_enum_check(int x_dtype, unsigned long long* pairs, unsigned long long* mismatches,
                         cudaStream_t stream) {
  if (x_dtype != HY3D_F16 && x_dtype != HY3D_BF16) return HY3D_ERR_ARG;
  if (!pairs || !mismatches) return HY3D_ERR_ARG;
  void* counts = nullptr;
  if (cudaGetSymbolAddress(&counts, g_enum_counts) != cudaSuccess) return HY3D_ERR_CUDA;
  if (cudaMemsetAsync(counts, 0, 2 * sizeof(unsigned long long), stream) != cudaSuccess)
    return HY3D_ERR_CUDA;
  if (x_dtype == HY3D_BF16) quotient_enum_kernel<true><<<32768, 256, 0, stream>>>();
  else quotient_enum_kernel<false><<<32768, 256, 0, stream>>>();
  if (cudaGetLastError() != cudaSuccess) return HY3D_ERR_CUDA;
  unsigned long long h[2] = {0, 0};
  if (cudaMemcpyAsync(h, counts, sizeof(h), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
    return HY3D_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return HY3D_ERR_CUDA;
  *pairs = h[0];
  *mismatches = h[1];
  return HY3D_OK;
}

int dequant_bias(const int32_t* acc, const float* act_scale, const void* w_scale, int ws_dtype,
                 const void* bias, int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N,
                 cudaStream_t stream) {
  if (!acc || !act_scale || !w_scale || !out) return HY3D_ERR_ARG;
  if (out_dtype != HY3D_F16 && out_dtype != HY3D_BF16) return HY3D_ERR_ARG;
  if (M < 0 || N <= 0 || (N & 7)) return HY3D_ERR_SHAPE;
  if (M == 0) return HY3D_OK;
  const int64_t total = M * (N >> 3);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  dequant_bias_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      acc, act_scale, w_scale, ws_dtype, bias, bias_dtype, out, out_dtype, M, N);
  return cudaGetLastError() == cudaSuccess ? HY3D_OK : HY3D_ERR_CUDA;
}

}  // namespace quant

using quant::quantize_rows;
using quant::layernorm_quantize;
using quant::dequant_bias;
using quant::quantizer_enum_check;

}  // namespace hy3d
