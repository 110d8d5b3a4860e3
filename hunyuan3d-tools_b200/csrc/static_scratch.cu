// Dense W8A8 linear layer for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where a layer runs: code
// executing inside a region where allocation is forbidden or would synchronise the device
// (a real-time render / capture loop, a plugin sandbox that only hands out pre-registered
// buffers, a process whose memory pool is owned by another runtime).  The regular entry
// point hy3d_linear_w8a8_dense needs two scratch buffers from its caller (the int8 copy of
// the activations and the per-token scales).  The entry point below takes only inputs and
// outputs and keeps that scratch in a fixed array that is part of the loaded library image,
// so every GPU that loads the library holds kStaticScratchBytes of it until the process
// exits.
//
// Rules that follow from the shared array:
//  * sizes are limited: M * K <= kStaticQBytes and M <= kStaticMaxRows, otherwise the call
//    returns HY3D_ERR_TOO_LARGE and launches nothing;
//  * the array keeps whatever the previous call left in it.  Nothing here needs to start at
//    zero: the quantise kernel of a call writes every byte (M*K codes, M scales) that the GEMM
//    of the same call reads, and rows past M are zero-filled by the tensor map, not read;
//  * all calls on one device share the array, so two calls whose kernels overlap on the GPU
//    (different streams, or different host threads without ordering) race.  Serialise them
//    on one stream;
//  * the first call on a device resolves the array's device address; make that first call
//    outside any stream capture.
#include "common.cuh"

#include <mutex>

namespace hy3d {
namespace static_scratch {

constexpr int64_t kStaticQBytes = 16ll << 20;          // quantised activations: up to 16 MiB
constexpr int64_t kStaticMaxRows = 65536;              // per-token scales: 256 KiB of floats
constexpr int64_t kStaticScratchBytes = kStaticQBytes + kStaticMaxRows * 4;

// In host code this name is only a handle for the runtime, not a device address; the
// address is obtained per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
std::mutex g_mutex;
void* g_scratch_addr[64] = {};

// Device address of the scratch array on the current device (resolved once per device).
int scratch_address(unsigned char** out) {
  const int dev = current_device();
  if (dev < 0 || dev >= 64) return HY3D_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return HY3D_ERR_CUDA;
    g_scratch_addr[dev] = ptr;
  }
  *out = static_cast<unsigned char*>(g_scratch_addr[dev]);
  return HY3D_OK;
}
}  // namespace

int linear_dense_static(const void* x, int x_dtype, int64_t ldx, const int8_t* B,
                        const void* w_scale, int ws_dtype, const void* bias, int bias_dtype,
                        void* out, int out_dtype, int64_t M, int64_t N, int64_t K, int epilogue,
                        cudaStream_t stream) {
  if (M < 0 || K <= 0 || N <= 0) return HY3D_ERR_SHAPE;
  // K is bounded first so that the product below cannot overflow.
  if (M > kStaticMaxRows || K > kStaticQBytes || M * K > kStaticQBytes) return HY3D_ERR_TOO_LARGE;
  unsigned char* base = nullptr;
  int rc = scratch_address(&base);
  if (rc != HY3D_OK) return rc;
  int8_t* q = reinterpret_cast<int8_t*>(base);
  float* scale = reinterpret_cast<float*>(base + kStaticQBytes);
  rc = quantize_rows(x, x_dtype, M, K, ldx, q, scale, stream);
  if (rc != HY3D_OK) return rc;
  return gemm_dense(q, B, scale, w_scale, ws_dtype, bias, bias_dtype, out, out_dtype, M, N, K,
                    epilogue, 0, 0, stream);
}

}  // namespace static_scratch
}  // namespace hy3d

extern "C" {

int hy3d_linear_w8a8_dense_static(const void* x, int x_dtype, int64_t ldx, const int8_t* B,
                                  const void* w_scale, int w_scale_dtype, const void* bias,
                                  int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N,
                                  int64_t K, int epilogue, void* stream) {
  const int rc = hy3d::check_device();
  if (rc != HY3D_OK) return rc;
  return hy3d::static_scratch::linear_dense_static(x, x_dtype, ldx, B, w_scale, w_scale_dtype, bias,
                                                   bias_dtype, out, out_dtype, M, N, K, epilogue,
                                                   static_cast<cudaStream_t>(stream));
}

int64_t hy3d_static_scratch_max_bytes(void) { return hy3d::static_scratch::kStaticQBytes; }
int64_t hy3d_static_scratch_max_rows(void) { return hy3d::static_scratch::kStaticMaxRows; }

}  // extern "C"
