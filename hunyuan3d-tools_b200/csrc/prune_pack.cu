// Offline 2:4 magnitude prune + compress + metadata pack for int8 weights, in one pass.
//
// Per group of four consecutive K elements the two smallest magnitudes are dropped with the
// reference's tie rule (strict comparisons, so on ties the later element survives) and the
// survivors are written in ascending index order together with the nibble idx0 | idx1<<2.
// One thread handles 32 consecutive K elements of one row: two 16-byte loads, one 16-byte
// store of compressed values, one 32-bit metadata word (8 nibbles, least-significant first)
// and optionally 8 raw nibble bytes.  Traffic: N*K read, N*K/2 + N*K/8 written.
#include "common.cuh"

namespace hy3d {
namespace prune {
namespace {

// Returns the nibble; writes the two survivors to k0,k1.
__device__ __forceinline__ uint32_t prune_group(const int (&v)[4], int& k0, int& k1) {
  int a[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) a[i] = v[i] < 0 ? -v[i] : v[i];
  int min1 = 0, min2 = 1;
  if (a[0] > a[1]) { min1 = 1; min2 = 0; }
#pragma unroll
  for (int i = 2; i < 4; ++i) {
    if (a[i] < a[min1]) { min2 = min1; min1 = i; }
    else if (a[i] < a[min2]) { min2 = i; }
  }
  int idx0 = -1, idx1 = -1;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i != min1 && i != min2) {
      if (idx0 < 0) idx0 = i; else idx1 = i;
    }
  }
  k0 = v[idx0];
  k1 = v[idx1];
  return static_cast<uint32_t>(idx0 | (idx1 << 2));
}

// The same selection without branches or indexed arrays, on the four bytes of one word: the
// dropped pair are the two smallest keys (|v|, index) -- the strict comparisons above keep the
// later element on ties, i.e. order equal magnitudes by index -- so element i survives iff at
// least two keys are smaller than its own.  Returns the nibble; `two` receives the survivors
// (ascending index) in its low 16 bits.
__device__ __forceinline__ uint32_t prune_word(uint32_t w, uint32_t& two) {
  const uint32_t a = __vabs4(w);                      // |v| per byte as unsigned (|-128| = 128)
  const uint32_t a0 = a & 0xFFu, a1 = (a >> 8) & 0xFFu, a2 = (a >> 16) & 0xFFu, a3 = a >> 24;
  // c_ij (i < j): key_i < key_j  <=>  a_i <= a_j
  const uint32_t c01 = a0 <= a1, c02 = a0 <= a2, c03 = a0 <= a3;
  const uint32_t c12 = a1 <= a2, c13 = a1 <= a3, c23 = a2 <= a3;
  const uint32_t r0 = 3u - c01 - c02 - c03;           // number of smaller keys
  const uint32_t r1 = 2u + c01 - c12 - c13;
  const uint32_t r2 = 1u + c02 + c12 - c23;
  const uint32_t r3 = c03 + c13 + c23;
  const uint32_t keep = (r0 >> 1) | ((r1 >> 1) << 1) | ((r2 >> 1) << 2) | ((r3 >> 1) << 3);
  const uint32_t idx0 = static_cast<uint32_t>(__ffs(static_cast<int>(keep)) - 1);
  const uint32_t idx1 = 31u - static_cast<uint32_t>(__clz(static_cast<int>(keep)));
  two = __byte_perm(w, 0u, idx0 | (idx1 << 4)) & 0xFFFFu;
  return idx0 | (idx1 << 2);
}

__device__ __forceinline__ void unpack4(uint32_t w, int (&v)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = static_cast<int>(static_cast<int8_t>((w >> (8 * i)) & 0xFF));
}

__global__ void __launch_bounds__(256)
prune_pack_kernel(const int8_t* __restrict__ w, int64_t N, int K, int8_t* __restrict__ comp,
                  uint8_t* __restrict__ meta_raw, uint32_t* __restrict__ meta_packed, int meta_ld) {
  const int chunks = K >> 5;                       // 32-wide K chunks that hold data
  const int per_row = meta_packed ? meta_ld : chunks;
  const int64_t total = N * per_row;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t row = idx / per_row;
  const int chunk = static_cast<int>(idx - row * per_row);
  if (chunk >= chunks) {  // padding word: any valid 2:4 pattern (indices 0,1)
    meta_packed[row * meta_ld + chunk] = 0x44444444u;
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(w + row * K + (chunk << 5));
  const uint4 lo = __ldcs(src), hi = __ldcs(src + 1);
  const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  uint32_t packed = 0;
  uint32_t out[4] = {0, 0, 0, 0};
  uint32_t raw[2] = {0, 0};
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    uint32_t two;
    const uint32_t nib = prune_word(words[g], two);
    packed |= nib << (4 * g);
    raw[g >> 2] |= nib << (8 * (g & 3));
    out[g >> 1] |= two << (16 * (g & 1));
  }
  *reinterpret_cast<uint4*>(comp + row * (K >> 1) + (chunk << 4)) =
      make_uint4(out[0], out[1], out[2], out[3]);
  if (meta_packed) meta_packed[row * meta_ld + chunk] = packed;
  if (meta_raw)
    *reinterpret_cast<uint2*>(meta_raw + row * (K >> 2) + (chunk << 3)) = make_uint2(raw[0], raw[1]);
}

// Any K % 4 == 0: one thread per group, byte accesses (small / odd matrices only).
__global__ void __launch_bounds__(256)
prune_compress_generic_kernel(const int8_t* __restrict__ w, int64_t N, int K,
                              int8_t* __restrict__ comp, uint8_t* __restrict__ meta_raw) {
  const int groups = K >> 2;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= N * groups) return;
  const int8_t* p = w + idx * 4;
  int v[4] = {p[0], p[1], p[2], p[3]}, k0, k1;
  const uint32_t nib = prune_group(v, k0, k1);
  comp[idx * 2] = static_cast<int8_t>(k0);
  comp[idx * 2 + 1] = static_cast<int8_t>(k1);
  if (meta_raw) meta_raw[idx] = static_cast<uint8_t>(nib);
}

}  // namespace

int prune_pack_24(const int8_t* w, int64_t N, int64_t K, int8_t* comp, uint8_t* meta_raw,
                  uint32_t* meta_packed, int64_t meta_ld, cudaStream_t stream) {
  if (!w || !comp) return HY3D_ERR_ARG;
  if (N < 0 || K <= 0 || (K & 3) || K > (1 << 20)) return HY3D_ERR_SHAPE;
  if (N == 0) return HY3D_OK;
  const bool fast = (K & 31) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(comp) & 15) == 0 &&
                    (!meta_raw || (reinterpret_cast<uintptr_t>(meta_raw) & 7) == 0);
  if (meta_packed) {
    if (!fast) return HY3D_ERR_SHAPE;
    if (meta_ld < (K >> 5)) return HY3D_ERR_SHAPE;
  }
  if (fast) {
    const int64_t per_row = meta_packed ? meta_ld : (K >> 5);
    const int64_t blocks = (N * per_row + 255) / 256;
    if (blocks > 0x7FFFFFFF) return HY3D_ERR_SHAPE;
    prune_pack_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        w, N, static_cast<int>(K), comp, meta_raw, meta_packed, static_cast<int>(meta_ld));
  } else {
    const int64_t blocks = (N * (K >> 2) + 255) / 256;
    if (blocks > 0x7FFFFFFF) return HY3D_ERR_SHAPE;
    prune_compress_generic_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        w, N, static_cast<int>(K), comp, meta_raw);
  }
  return cudaGetLastError() == cudaSuccess ? HY3D_OK : HY3D_ERR_CUDA;
}

}  // namespace prune

using prune::prune_pack_24;

}  // namespace hy3d
