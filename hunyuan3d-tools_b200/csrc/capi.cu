// C ABI of libhy3d_int8.so: argument checks, tensor-map encoding and dispatch to the
// kernels.  No allocation happens behind these entry points.
#include "common.cuh"

#include <cudaTypedefs.h>
#include <mutex>

namespace hy3d {

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices];
int g_cc_major[kMaxDevices];
bool g_dev_known[kMaxDevices];
std::mutex g_dev_mutex;

int query_device(int* sm_count, int* cc_major) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HY3D_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return HY3D_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_dev_known[dev]) {
    int sms = 0, major = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
      return HY3D_ERR_CUDA;
    g_sm_count[dev] = sms;
    g_cc_major[dev] = major;
    g_dev_known[dev] = true;
  }
  *sm_count = g_sm_count[dev];
  *cc_major = g_cc_major[dev];
  return HY3D_OK;
}

int check_device() {
  int sms = 0, major = 0;
  const int rc = query_device(&sms, &major);
  if (rc != HY3D_OK) return rc;
  return major == 10 ? HY3D_OK : HY3D_ERR_DEVICE;
}

}  // namespace

int device_sm_count() {
  int sms = 0, major = 0;
  return query_device(&sms, &major) == HY3D_OK ? sms : -1;
}

int current_device() {
  int dev = 0;
  return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}

// Kernels here ask for more dynamic shared memory than the default limit; the attribute is
// set once per (device, kernel).  Callers may launch from several host threads.
int ensure_max_smem(const void* kernel, int bytes) {
  constexpr int kSlots = 256;
  static std::mutex mu;
  static const void* seen_fn[kSlots];
  static int seen_dev[kSlots];
  static int n_seen = 0;
  const int dev = current_device();
  if (dev < 0) return HY3D_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_seen; ++i)
    if (seen_fn[i] == kernel && seen_dev[i] == dev) return HY3D_OK;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    cudaGetLastError();
    return HY3D_ERR_CUDA;
  }
  if (n_seen < kSlots) {
    seen_fn[n_seen] = kernel;
    seen_dev[n_seen] = dev;
    ++n_seen;
  }
  return HY3D_OK;
}

// 2-D byte tensor: `rows` rows of `inner_bytes` bytes, `pitch_bytes` apart; the box is
// box_inner bytes x box_rows rows.  Out-of-range parts of a box read as zero.
int encode_tmap_2d_u8(CUtensorMap* map, const void* base, uint64_t inner_bytes, uint64_t rows,
                      uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows,
                      int swizzle_bytes) {
  EncodeFn fn = get_encode_fn();
  if (!fn) return HY3D_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15)) return HY3D_ERR_SHAPE;
  if (box_inner == 0 || box_rows == 0 || box_inner > 256 || box_rows > 256) return HY3D_ERR_SHAPE;
  const cuuint64_t dims[2] = {inner_bytes, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = swizzle_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                                : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                      : CU_TENSOR_MAP_SWIZZLE_NONE;
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? HY3D_OK : HY3D_ERR_CUDA;
}

}  // namespace hy3d

using namespace hy3d;

extern "C" {

#ifdef HY3D_TRACE
// Diagnostic builds only: copies out and clears the timeline of the traced CTA.
int hy3d_trace_read(unsigned long long* out, int next_cta) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out, g_trace_buf, 4 * 4096 * sizeof(unsigned long long));
  static unsigned long long zeros[4 * 4096];
  cudaMemcpyToSymbol(g_trace_buf, zeros, sizeof(zeros));
  cudaMemcpyToSymbol(g_trace_cta, &next_cta, sizeof(int));
  return 0;
}
#endif

// Bumped whenever an entry point's argument list or meaning changes; the Python binding
// refuses a library whose number differs from the one it was written against.
int hy3d_version(void) { return HY3D_ABI_VERSION; }
#ifndef HY3D_SOURCE_DIGEST
#define HY3D_SOURCE_DIGEST "unknown"
#endif
const char* hy3d_source_digest(void) { return HY3D_SOURCE_DIGEST; }
const char* hy3d_arch(void) { return "sm_100a"; }

const char* hy3d_status_string(int status) {
  switch (status) {
    case HY3D_OK: return "ok";
    case HY3D_ERR_ARG: return "bad argument (null pointer or unknown enum)";
    case HY3D_ERR_SHAPE: return "unsupported size, divisibility or alignment";
    case HY3D_ERR_CUDA: return "CUDA call failed";
    case HY3D_ERR_DEVICE: return "device is not compute capability 10.x";
    case HY3D_ERR_TIMEOUT: return "device-side wait timed out";
    case HY3D_ERR_TOO_LARGE: return "size exceeds a fixed internal capacity";
    default: return "unknown status";
  }
}

int hy3d_last_device_status(int* status_out) {
  if (!status_out) return HY3D_ERR_ARG;
  if (cudaDeviceSynchronize() != cudaSuccess) return HY3D_ERR_CUDA;
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return HY3D_ERR_CUDA;
  if (v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)) != cudaSuccess) return HY3D_ERR_CUDA;
  }
  *status_out = v;
  return HY3D_OK;
}

int hy3d_groupnorm_nhwc(const void* x, const void* add, int x_dtype, int64_t B, int64_t HW, int64_t C,
                        int groups, const void* gamma, const void* beta, int gb_dtype, float eps,
                        int silu, void* y, float* workspace, void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  return gnorm::groupnorm_nhwc(x, add, x_dtype, B, HW, C, groups, gamma, beta, gb_dtype, eps, silu, y,
                               workspace, static_cast<cudaStream_t>(stream));
}

int64_t hy3d_groupnorm_workspace_floats(int64_t B, int64_t HW, int groups) {
  if (B <= 0 || HW <= 0 || groups <= 0) return 0;
  return gnorm::workspace_floats(B, HW, groups);
}

int hy3d_stream_status(void* stream) {
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) return HY3D_ERR_CUDA;
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return HY3D_ERR_CUDA;
  return v == 0 ? HY3D_OK : HY3D_ERR_TIMEOUT;
}

int hy3d_set_wait_limit_ns(unsigned long long limit_ns) {
  if (limit_ns == 0) limit_ns = kWaitLimitNs;
  if (cudaMemcpyToSymbol(g_wait_limit_ns, &limit_ns, sizeof(limit_ns)) != cudaSuccess)
    return HY3D_ERR_CUDA;
  return HY3D_OK;
}

int hy3d_wait_selftest(void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>();
  return cudaGetLastError() == cudaSuccess ? HY3D_OK : HY3D_ERR_CUDA;
}

int hy3d_quantize_rows(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* q,
                       float* scale, void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  return quantize_rows(x, x_dtype, M, K, ldx, q, scale, static_cast<cudaStream_t>(stream));
}

int hy3d_layernorm_quantize(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                            const void* gamma, const void* beta, int gb_dtype, float eps, int8_t* q,
                            float* scale, void* y_out, void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  return layernorm_quantize(x, x_dtype, M, K, ldx, gamma, beta, gb_dtype, eps, q, scale, y_out,
                            static_cast<cudaStream_t>(stream));
}

int hy3d_quantizer_enum_check(int x_dtype, unsigned long long* pairs_out,
                              unsigned long long* mismatches_out, void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  return quantizer_enum_check(x_dtype, pairs_out, mismatches_out, static_cast<cudaStream_t>(stream));
}

int hy3d_gemm_w8a8_dense(const int8_t* A, const int8_t* B, const float* act_scale,
                         const void* w_scale, int w_scale_dtype, const void* bias, int bias_dtype,
                         void* out, int out_dtype, int64_t M, int64_t N, int64_t K, int epilogue,
                         int cta_group, int block_n, void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  return gemm_dense(A, B, act_scale, w_scale, w_scale_dtype, bias, bias_dtype, out, out_dtype, M,
                    N, K, epilogue, cta_group, block_n, static_cast<cudaStream_t>(stream));
}

int hy3d_dense_splitk_plan(int64_t M, int64_t N, int64_t K, int epilogue, int64_t* workspace_bytes) {
  if (check_device() != HY3D_OK) return 1;
  const int splits = dense_splitk_plan(M, N, K, epilogue);
  // every K range owns an M-padded (whole 128-row tiles) int32 matrix
  if (workspace_bytes) *workspace_bytes = splits > 1 ? static_cast<int64_t>(splits) * ((M + 127) / 128 * 128) * N * 4 : 0;
  return splits;
}

int hy3d_gemm_w8a8_dense_splitk(const int8_t* A, const int8_t* B, const float* act_scale,
                                const void* w_scale, int w_scale_dtype, const void* bias,
                                int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N,
                                int64_t K, int epilogue, int splits, void* workspace,
                                int64_t workspace_bytes, void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  if (splits < 1 || splits > 64) return HY3D_ERR_ARG;
  if (splits > 1 && (!workspace || workspace_bytes < static_cast<int64_t>(splits) * ((M + 127) / 128 * 128) * N * 4))
    return HY3D_ERR_TOO_LARGE;
  return gemm_dense(A, B, act_scale, w_scale, w_scale_dtype, bias, bias_dtype, out, out_dtype, M,
                    N, K, epilogue, splits > 1 ? 1 : 0, 0, static_cast<cudaStream_t>(stream), splits,
                    static_cast<int32_t*>(workspace));
}

int hy3d_linear_w8a8_dense(const void* x, int x_dtype, int64_t ldx, int8_t* q_ws, float* scale_ws,
                           const int8_t* B, const void* w_scale, int w_scale_dtype,
                           const void* bias, int bias_dtype, void* out, int out_dtype, int64_t M,
                           int64_t N, int64_t K, int epilogue, int cta_group, int block_n,
                           void* stream) {
  int rc = check_device();
  if (rc != HY3D_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // One launch with the quantised activations resident in shared memory where that is the
  // faster path (and the caller left tile shape and grouping to the library); same bits.
  if (cta_group == 0 && block_n == 0 && x_dtype == out_dtype && (ldx & 7) == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      linear_path(M, K, N, epilogue) == 1)
    return linear_fused(x, x_dtype, ldx, nullptr, B, w_scale, w_scale_dtype, bias, bias_dtype, out,
                        out_dtype, M, N, K, epilogue, 0, s);
  rc = quantize_rows(x, x_dtype, M, K, ldx, q_ws, scale_ws, s);
  if (rc != HY3D_OK) return rc;
  return gemm_dense(q_ws, B, scale_ws, w_scale, w_scale_dtype, bias, bias_dtype, out, out_dtype, M,
                    N, K, epilogue, cta_group, block_n, s);
}

int hy3d_linear_path(int64_t M, int64_t K, int64_t N, int epilogue) {
  if (check_device() != HY3D_OK) return 0;
  return linear_path(M, K, N, epilogue);
}

int hy3d_linear_w8a8_dense_fused(const void* x, int x_dtype, int64_t ldx, float* scale_out,
                                 const int8_t* B, const void* w_scale, int w_scale_dtype,
                                 const void* bias, int bias_dtype, void* out, int out_dtype,
                                 int64_t M, int64_t N, int64_t K, int epilogue, int block_n,
                                 void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  return linear_fused(x, x_dtype, ldx, scale_out, B, w_scale, w_scale_dtype, bias, bias_dtype, out,
                      out_dtype, M, N, K, epilogue, block_n, static_cast<cudaStream_t>(stream));
}

int hy3d_prune_pack_24(const int8_t* w, int64_t N, int64_t K, int8_t* comp, uint8_t* meta_raw,
                       uint32_t* meta_packed, int64_t meta_ld, void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  return prune_pack_24(w, N, K, comp, meta_raw, meta_packed, meta_ld,
                       static_cast<cudaStream_t>(stream));
}

int hy3d_gemm_w8a8_sparse24(const int8_t* X, const float* act_scale, const int8_t* w_comp,
                            const uint32_t* w_meta, int64_t meta_ld, const void* w_scale,
                            int w_scale_dtype, const void* bias, int bias_dtype, void* out,
                            int out_dtype, int64_t M, int64_t N, int64_t K, int epilogue,
                            int block_m, void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  return gemm_sparse24(X, act_scale, w_comp, w_meta, meta_ld, w_scale, w_scale_dtype, bias,
                       bias_dtype, out, out_dtype, M, N, K, epilogue, block_m,
                       static_cast<cudaStream_t>(stream));
}

int hy3d_linear_w8a8_sparse24(const void* x, int x_dtype, int64_t ldx, int8_t* q_ws,
                              float* scale_ws, const int8_t* w_comp, const uint32_t* w_meta,
                              int64_t meta_ld, const void* w_scale, int w_scale_dtype,
                              const void* bias, int bias_dtype, void* out, int out_dtype,
                              int64_t M, int64_t N, int64_t K, int epilogue, int block_m,
                              void* stream) {
  int rc = check_device();
  if (rc != HY3D_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  rc = quantize_rows(x, x_dtype, M, K, ldx, q_ws, scale_ws, s);
  if (rc != HY3D_OK) return rc;
  return gemm_sparse24(q_ws, scale_ws, w_comp, w_meta, meta_ld, w_scale, w_scale_dtype, bias,
                       bias_dtype, out, out_dtype, M, N, K, epilogue, block_m, s);
}

int hy3d_dequant_bias(const int32_t* acc, const float* act_scale, const void* w_scale,
                      int w_scale_dtype, const void* bias, int bias_dtype, void* out,
                      int out_dtype, int64_t M, int64_t N, void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  return dequant_bias(acc, act_scale, w_scale, w_scale_dtype, bias, bias_dtype, out, out_dtype, M,
                      N, static_cast<cudaStream_t>(stream));
}

int hy3d_mma_kat(const int8_t* a, const int8_t* b, const uint32_t* meta, int32_t* d, int n,
                 int ksteps, int sparse, void* stream) {
  const int rc = check_device();
  if (rc != HY3D_OK) return rc;
  if (!a || !b || !d) return HY3D_ERR_ARG;
  if (n < 16 || n > 256 || (n & 15)) return HY3D_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!sparse) {
    if (ksteps < 1 || ksteps > 4) return HY3D_ERR_SHAPE;
    // D(128 x n) = A(128 x k) * B(n x k)^T: the dense GEMM with exactly one tile.
    return gemm_dense(a, b, nullptr, nullptr, HY3D_F32, nullptr, HY3D_F32, d, HY3D_S32, 128, n,
                      32 * ksteps, HY3D_EPI_LINEAR, 1, n, s);
  }
  if (!meta) return HY3D_ERR_ARG;
  if (ksteps < 1 || ksteps > 2) return HY3D_ERR_SHAPE;
  // The sparse GEMM computes out(M = tokens, N = weight rows); here the 128 compressed rows
  // are the weight and the n rows of b are the tokens, so d receives D^T, (n, 128) row-major
  // (as the header says); the binding transposes it back.
  const int64_t k = 64 * ksteps;
  return gemm_sparse24(b, nullptr, a, meta, 4 * ((k + 127) / 128), nullptr, HY3D_F32, nullptr,
                       HY3D_F32, d, HY3D_S32, n, 128, k, HY3D_EPI_LINEAR, n, s);
}

}  // extern "C"
