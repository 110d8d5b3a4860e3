/*
 * hy3d_int8.h -- C ABI of the sm_100a W8A8 linear-layer library (libhy3d_int8.so).
 *
 * Every entry point takes raw device pointers, 64-bit sizes, small enums and a CUDA
 * stream passed as `void*` (a cudaStream_t); it returns 0 on success or one of the
 * HY3D_ERR_* codes below.  Nothing here allocates device memory: the caller owns all
 * inputs, outputs and workspaces.  No C++ or torch type crosses this boundary.
 *
 * Each declaration cites the interface of WizardsForgeGames/Hunyuan3D-Tools that it
 * stands in for (path within that project : lines).
 */
#ifndef HY3D_INT8_H_
#define HY3D_INT8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------ */
#define HY3D_OK               0
#define HY3D_ERR_ARG          1  /* null pointer, unknown enum value                      */
#define HY3D_ERR_SHAPE        2  /* size / divisibility / alignment rule violated         */
#define HY3D_ERR_CUDA         3  /* a CUDA runtime or driver call failed                  */
#define HY3D_ERR_DEVICE       4  /* device is not compute capability 10.x                 */
#define HY3D_ERR_TIMEOUT      5  /* a bounded device-side wait gave up (see last_status)  */
#define HY3D_ERR_TOO_LARGE    6  /* size exceeds a fixed internal capacity                */

/* ---- element types ------------------------------------------------------------------ */
#define HY3D_F16   0
#define HY3D_BF16  1
#define HY3D_F32   2   /* scales / bias only                                              */
#define HY3D_S32   3   /* GEMM output only: raw int32 accumulators, no rescale            */

/* ---- GEMM epilogues ------------------------------------------------------------------ */
#define HY3D_EPI_LINEAR  0  /* y = acc * (act_scale[m] * w_scale[n]) + bias[n]             */
#define HY3D_EPI_GELU    1  /* y = gelu_erf(linear)                                        */
#define HY3D_EPI_GEGLU   2  /* weights row-interleaved in blocks of 16 (value,gate):
                               y[m, j] = value * gelu_erf(gate); output has N/2 columns   */

/* ABI version (changes whenever an argument list or its meaning does), build architecture
 * ("sm_100a") and the digest of the sources the library was built from. */
int         hy3d_version(void);
const char* hy3d_arch(void);
const char* hy3d_source_digest(void);
const char* hy3d_status_string(int status);

/* Reads (with a device synchronisation) and clears the device-side error word that a
 * kernel sets when one of its bounded waits ran out.  0 = no error recorded. */
int hy3d_last_device_status(int* status_out);

/* Waits for `stream` and returns HY3D_ERR_TIMEOUT if a kernel has recorded a bounded wait
 * that ran out since the error word was last cleared (the output of that launch is then
 * undefined), HY3D_OK otherwise.  Does not clear the word; hy3d_last_device_status does. */
int hy3d_stream_status(void* stream);

/* Test hooks of the bounded waits (no reference counterpart).  hy3d_set_wait_limit_ns sets the
 * longest any device-side wait may last on the current device (0 restores the default of 2 s);
 * hy3d_wait_selftest launches one thread that waits on a barrier nobody signals, so that the
 * limit runs out, the error word is set and the kernel returns normally. */
int hy3d_set_wait_limit_ns(unsigned long long limit_ns);
int hy3d_wait_selftest(void* stream);

/*
 * Per-token (per-row) symmetric absmax quantisation: for each of the M rows
 *     scale = max(max_k |x|, 1e-8) / 127 ;  q = clamp(rint(x / scale), -128, 127)
 * x: (M,K) f16 or bf16, row pitch ldx elements.  q: (M,K) int8 contiguous.  scale: (M) f32.
 * Requires K % 8 == 0, K <= 16384, 16-byte aligned x rows.
 * Replaces: csrc/int8_gemm_tc.cu:190-242 (_tc_fused_quantize), csrc/int8_kernels.cu:26-88,
 * 128-153 (fused_quantize_activation), csrc/int8_sparse_tc.cu:218-336, 1668-1707
 * (sparse_quantize_act).
 */
int hy3d_quantize_rows(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                       int8_t* q, float* scale, void* stream);

/*
 * LayerNorm over the last dimension fused with the per-token quantiser above: the row is
 * normalised in registers, rounded to x_dtype exactly as a stand-alone LayerNorm would store
 * it, and the rounded values are quantised -- q and scale equal
 * hy3d_quantize_rows(LayerNorm(x)) bit for bit and the normalised activations never go to
 * memory.  gamma / beta: (K) of gb_dtype (f16/bf16/f32) or NULL (1 / 0).  y_out: optional
 * (M,K) x_dtype array that receives the rounded LayerNorm output, or NULL.
 * Arithmetic (fp32): mean = sum(x)/K; var = sum((x-mean)^2)/K; rstd = 1/sqrt(var+eps) with IEEE
 * square root and reciprocal; y = fma((x-mean)*rstd, gamma, beta).  Requires K % 8 == 0,
 * K <= 2048, 16-byte aligned rows.
 * Replaces nothing in the reference by itself: the reference's layers re-quantise the
 * LayerNorm output for every sibling projection (csrc/int8_sparse_tc.cu:269-271 notes the
 * re-reads); this is the producer-side emission that removes that pass.  Its consumers are
 * hy3d_gemm_w8a8_dense / hy3d_gemm_w8a8_sparse24.
 */
int hy3d_layernorm_quantize(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                            const void* gamma, const void* beta, int gb_dtype, float eps,
                            int8_t* q, float* scale, void* y_out, void* stream);

/*
 * GroupNorm (+ optional SiLU) over channels-last activations: x and y are (B, HW, C) arrays of
 * x_dtype (f16/bf16) with C contiguous -- the memory of a torch channels_last (B, C, H, W)
 * tensor -- groups are runs of C / groups adjacent channels, statistics are taken over
 * HW x C / groups elements per (sample, group) in fp32 (sum and sum of squares, fixed summation
 * order).  y = x * (rstd * gamma[c]) + (beta[c] - mean * rstd * gamma[c]) rounded to x_dtype;
 * with silu != 0 the rounded value v becomes v / (1 + exp(-v)), rounded again.  gamma / beta:
 * (C) of gb_dtype or NULL.  workspace: hy3d_groupnorm_workspace_floats(B, HW, groups) floats of
 * device memory owned by the caller (per-chunk partial sums; no initialisation needed).
 * add: optional (B, C) array of x_dtype added to every pixel of its sample before the
 * normalisation -- x + add[b, c] rounded to x_dtype, as a separate broadcast add would store it
 * (a UNet's time-embedding term) -- or NULL.
 * Requires C % 8 == 0, C % groups == 0, C <= 2560, 16-byte aligned x, y and add.  y may equal x.
 * Replaces nothing in the reference (its UNet normalises with stock PyTorch); it serves the
 * model around the INT8 layers, whose convolutions run NHWC while torch's GroupNorm kernel
 * takes NCHW only and so costs two layout copies per call.
 */
int hy3d_groupnorm_nhwc(const void* x, const void* add, int x_dtype, int64_t B, int64_t HW, int64_t C,
                        int groups, const void* gamma, const void* beta, int gb_dtype, float eps,
                        int silu, void* y, float* workspace, void* stream);
int64_t hy3d_groupnorm_workspace_floats(int64_t B, int64_t HW, int groups);

/*
 * Self-check of the quantiser's rounding (test hook, no reference counterpart).  The kernel
 * above never divides; this call enumerates on the device every pair of 16-bit patterns
 * (amax, x) of x_dtype with |x| <= amax -- every input the quantiser can meet -- and counts the
 * pairs whose code differs from (int8) rint(x / scale) computed with IEEE divisions.
 * Synchronises the stream; *mismatches_out must come back 0 (about 1e9 pairs, ~0.1 s).
 */
int hy3d_quantizer_enum_check(int x_dtype, unsigned long long* pairs_out,
                              unsigned long long* mismatches_out, void* stream);

/*
 * Dense W8A8 GEMM with fused epilogue.
 *   acc[m,n] = sum_k A[m,k] * B[n,k]          (int32, exact)
 *   out      = epilogue(acc, act_scale, w_scale, bias)  in out_dtype (f16 / bf16), or the
 *              raw accumulators when out_dtype == HY3D_S32 (scales and bias ignored).
 * A: (M,K) int8 row-major.  B: (N,K) int8 row-major.  act_scale: (M) f32.
 * w_scale: (N) of w_scale_dtype (f16/bf16/f32).  bias: (N) of bias_dtype, or NULL.
 * out: (M, N) -- (M, N/2) for HY3D_EPI_GEGLU -- row-major, contiguous.
 * Requires K % 16 == 0, N % 16 == 0 (N % 32 for GEGLU), 16-byte aligned pointers.
 * cta_group: 0 = choose, 1 = one CTA per tile, 2 = CTA pair (256-row tiles).
 * block_n:   0 = choose, else the tile width (multiple of 16, <= 256).
 * Replaces: csrc/int8_gemm_tc.cu:36-184, 254-309 (int8_gemm_tc) and the epilogue-only
 * kernel csrc/int8_kernels.cu:99-121 (fused_dequantize_bias) that followed torch::_int_mm.
 */
int hy3d_gemm_w8a8_dense(const int8_t* A, const int8_t* B, const float* act_scale,
                         const void* w_scale, int w_scale_dtype,
                         const void* bias, int bias_dtype,
                         void* out, int out_dtype,
                         int64_t M, int64_t N, int64_t K,
                         int epilogue, int cta_group, int block_n, void* stream);

/*
 * Split-K form of the GEMM above for launches whose tiles leave most SMs idle while each walks
 * a long K alone (few rows, deep K: the image encoder's M = 257, K = 6144 layer): the K blocks
 * are cut into `splits` ranges that run side by side as int32 partials in `workspace`
 * (splits x ceil(M/128)*128 x N x 4 bytes, 16-byte aligned, no initialisation needed), and a second kernel
 * adds the partials -- exactly, in int32 -- and applies the epilogue with the GEMM kernel's own
 * formula and roundings, so the result equals hy3d_gemm_w8a8_dense bit for bit.
 * hy3d_dense_splitk_plan returns the number of ranges this library would use for a shape
 * (1 = do not split) and the workspace it needs.  out_dtype f16/bf16, epilogue linear or GELU,
 * N % 8 == 0; splits = 1 runs the plain kernel.
 * Replaces: the split-K path and its reduce kernel of the reference's sparse GEMM
 * (csrc/int8_sparse_tc.cu:1730-1732 cost terms, split-K reduce) in the dense kernel's terms.
 */
int hy3d_dense_splitk_plan(int64_t M, int64_t N, int64_t K, int epilogue, int64_t* workspace_bytes);
int hy3d_gemm_w8a8_dense_splitk(const int8_t* A, const int8_t* B, const float* act_scale,
                                const void* w_scale, int w_scale_dtype,
                                const void* bias, int bias_dtype,
                                void* out, int out_dtype,
                                int64_t M, int64_t N, int64_t K,
                                int epilogue, int splits, void* workspace, int64_t workspace_bytes,
                                void* stream);

/*
 * Whole dense linear layer: quantise x per token into the caller's workspace, then the
 * GEMM above.  x: (M,K) f16/bf16; q_ws: (M,K) int8 workspace; scale_ws: (M) f32 workspace.
 * Replaces: csrc/int8_gemm_tc.cu:312-320 (int8_linear_tc), csrc/int8_kernels.cu:193-210
 * (int8_linear_fused).
 */
int hy3d_linear_w8a8_dense(const void* x, int x_dtype, int64_t ldx,
                           int8_t* q_ws, float* scale_ws,
                           const int8_t* B, const void* w_scale, int w_scale_dtype,
                           const void* bias, int bias_dtype,
                           void* out, int out_dtype,
                           int64_t M, int64_t N, int64_t K,
                           int epilogue, int cta_group, int block_n, void* stream);

/*
 * The same layer as ONE kernel with the quantised activations resident in shared memory: a
 * CTA quantises a block of 128 tokens straight into the swizzled operand tiles of the whole K
 * and runs every weight tile assigned to it against that block, so the int8 activations never
 * exist in global memory and the layer moves 2*M*K + N*K + 2*M*N bytes.  Results are
 * bit-identical to hy3d_linear_w8a8_dense.  Needs x_dtype == out_dtype (f16 / bf16),
 * K % 32 == 0, K <= 1280, ldx % 8 == 0, N % 16 == 0 (N % 32 for GEGLU) and 16-byte aligned
 * pointers; anything else returns HY3D_ERR_SHAPE / HY3D_ERR_ARG and launches nothing.
 * scale_out: optional (M) f32 array that receives the per-token scales, or NULL.
 * block_n: 0 = choose, else the weight-tile width (multiple of 32, 64 for GEGLU, <= 256).
 * hy3d_linear_w8a8_dense takes this path by itself for the shapes where it is the faster one;
 * hy3d_linear_path(M, K, N, epilogue) tells which (1 = one launch, 0 = two launches).
 * Replaces: the fused quantise + GEMM path csrc/int8_sparse_tc.cu:657-734, 1934-2002
 * (sparse_gemm_fq_kernel, sp_use_fused, sparse_fq_launch) and the path query
 * csrc/int8_sparse_tc.cu:2065-2070 (sparse_int8_linear_path), for the dense layer.
 */
int hy3d_linear_w8a8_dense_fused(const void* x, int x_dtype, int64_t ldx, float* scale_out,
                                 const int8_t* B, const void* w_scale, int w_scale_dtype,
                                 const void* bias, int bias_dtype,
                                 void* out, int out_dtype,
                                 int64_t M, int64_t N, int64_t K,
                                 int epilogue, int block_n, void* stream);
int hy3d_linear_path(int64_t M, int64_t K, int64_t N, int epilogue);

/*
 * The dense linear layer again, for callers that may not allocate device memory where the
 * layer runs (an allocation-free region of a render or capture loop, a sandboxed plugin that
 * is only handed pre-registered buffers, a process whose device pool belongs to another
 * runtime): the two scratch buffers hy3d_linear_w8a8_dense asks for live in a fixed array
 * inside the library instead, so only inputs and outputs are passed.  No counterpart in the
 * reference, whose extension allocates its scratch through torch on every call.
 * Limits: M * K <= hy3d_static_scratch_max_bytes() (16 MiB) and
 * M <= hy3d_static_scratch_max_rows() (65536); beyond them the call returns
 * HY3D_ERR_TOO_LARGE and launches nothing.  Every GPU that loads the library holds that array
 * (16.25 MiB) until the process exits.  Calls on one device share it: run them on one stream,
 * since calls whose kernels overlap on the GPU race on it.  Its contents carry over between
 * calls, which is harmless: each call overwrites everything it later reads.  The first call on
 * a device looks up the array's device address; make that call before any stream capture.
 * Tile shape and CTA grouping are chosen by the library (as with 0 / 0 in the regular call).
 */
int hy3d_linear_w8a8_dense_static(const void* x, int x_dtype, int64_t ldx,
                                  const int8_t* B, const void* w_scale, int w_scale_dtype,
                                  const void* bias, int bias_dtype,
                                  void* out, int out_dtype,
                                  int64_t M, int64_t N, int64_t K,
                                  int epilogue, void* stream);
int64_t hy3d_static_scratch_max_bytes(void);
int64_t hy3d_static_scratch_max_rows(void);

/*
 * Offline 2:4 prune + compress + metadata pack of an int8 weight matrix, one pass.
 * Per group of 4 along K the two smallest |w| are dropped; the tie rule is
 *   min1=0,min2=1; if |w0|>|w1| swap; for i in 2,3: if |wi|<|w[min1]| {min2=min1;min1=i}
 *   else if |wi|<|w[min2]| {min2=i}      (both comparisons strict)
 * and the survivors keep ascending index order (idx0 < idx1).
 * w: (N,K) int8.  comp: (N,K/2) int8.  meta_raw (optional, may be NULL): (N*K/4) bytes,
 * one nibble idx0 | idx1<<2 per group.  meta_packed (optional): (N, meta_ld) uint32 words,
 * word c of a row = the 8 nibbles of K chunk [32c, 32c+32), least-significant first;
 * meta_ld >= K/32, words [K/32, meta_ld) of each row are written as 0x44444444.
 * Requires K % 4 == 0; with meta_packed also K % 32 == 0 and 16-byte aligned w and comp
 * (8-byte aligned meta_raw).  Matrices that meet the second rule take the vectorised kernel.
 * Replaces: csrc/int8_sparse_tc.cu:152-212 (prune_compress_kernel), 416-437
 * (pack_metadata_kernel), 1558-1585 (sparse_prune_compress), 1616-1665
 * (sparse_prune_and_pack).
 */
int hy3d_prune_pack_24(const int8_t* w, int64_t N, int64_t K,
                       int8_t* comp, uint8_t* meta_raw,
                       uint32_t* meta_packed, int64_t meta_ld, void* stream);

/*
 * 2:4 structured-sparse W8A8 GEMM with the same epilogues as the dense one.
 *   acc[m,n] = sum_k X[m,k] * Wpruned[n,k]
 * X: (M,K) int8.  w_comp: (N,K/2) int8.  w_meta: (N, meta_ld) uint32 as written by
 * hy3d_prune_pack_24 with meta_ld = 4*ceil(K/128).  Other arguments as for the dense GEMM.
 * Requires K % 64 == 0, N % 16 == 0.  block_m: 0 = choose, else the token-tile width
 * (multiple of 16, <= 256).
 * Replaces: csrc/int8_sparse_tc.cu:535-1123, 1758-1929 (sparse_int8_gemm) and 519-531
 * (splitk_reduce_kernel; there is no split-K here, accumulation stays int32).
 */
int hy3d_gemm_w8a8_sparse24(const int8_t* X, const float* act_scale,
                            const int8_t* w_comp, const uint32_t* w_meta, int64_t meta_ld,
                            const void* w_scale, int w_scale_dtype,
                            const void* bias, int bias_dtype,
                            void* out, int out_dtype,
                            int64_t M, int64_t N, int64_t K,
                            int epilogue, int block_m, void* stream);

/*
 * Whole sparse linear layer: quantise + sparse GEMM.
 * Replaces: csrc/int8_sparse_tc.cu:2006-2044 (sparse_int8_linear, sparse_int8_linear_ex).
 */
int hy3d_linear_w8a8_sparse24(const void* x, int x_dtype, int64_t ldx,
                              int8_t* q_ws, float* scale_ws,
                              const int8_t* w_comp, const uint32_t* w_meta, int64_t meta_ld,
                              const void* w_scale, int w_scale_dtype,
                              const void* bias, int bias_dtype,
                              void* out, int out_dtype,
                              int64_t M, int64_t N, int64_t K,
                              int epilogue, int block_m, void* stream);

/*
 * Epilogue-only kernel on an int32 accumulator matrix:
 *   out[m,n] = acc[m,n] * (act_scale[m] * w_scale[n]) + bias[n]
 * Replaces: csrc/int8_kernels.cu:99-121, 156-190 (fused_dequantize_bias).
 */
int hy3d_dequant_bias(const int32_t* acc, const float* act_scale,
                      const void* w_scale, int w_scale_dtype,
                      const void* bias, int bias_dtype,
                      void* out, int out_dtype, int64_t M, int64_t N, void* stream);

/*
 * Known-answer hook: ONE tensor-core tile product on a single CTA.
 *   sparse == 0: D(128 x n) = A(128 x k) * B(n x k)^T, k = 32 * ksteps  (tcgen05.mma kind::i8)
 *   sparse == 1: A is 2:4 compressed (128 x k/2) with meta (128 x 4*ceil(k/128)) words,
 *                k = 64 * ksteps                                 (tcgen05.mma.sp kind::i8)
 * n: multiple of 16 in [16,256]; ksteps in [1,4] (dense) or [1,2] (sparse).
 * d: int32, (128, n) row-major for the dense case; for the sparse case the tile is written
 * transposed, (n, 128) row-major (the sparse kernel's accumulator is D[weight row, token] and
 * its output is token-major).
 * Replaces: csrc/int8_sparse_tc.cu:350-408, 1587-1614 (test_mma_sp).
 */
int hy3d_mma_kat(const int8_t* a, const int8_t* b, const uint32_t* meta,
                 int32_t* d, int n, int ksteps, int sparse, void* stream);

/*
 * Measurement hooks (no reference counterpart; never on the layer path).
 * hy3d_probe_mma_i8: one CTA per SM issues `groups` groups of four tcgen05.mma kind::i8
 *   (128 x n x 32, or the 2:4-sparse 128 x n x 64 form when sparse != 0) on operands that stay
 *   in shared memory, with the commit / wait cadence of a two-stage pipeline and no loads;
 *   *ops_out receives the dense-equivalent operation count of the launch (2*M*N*K summed), so
 *   ops / elapsed time is the tensor throughput this GPU sustains for that instruction.
 * hy3d_probe_hbm: streams `bytes` (a multiple of 16) of the caller's buffer `a` with 16-byte
 *   accesses from every SM: mode 0 writes it, mode 1 reads it, mode 2 copies it to `b`.
 */
int hy3d_probe_mma_i8(int n, int groups, int sparse, int64_t* ops_out, void* stream);
int hy3d_probe_hbm(int mode, void* a, void* b, int64_t bytes, void* stream);

/*
 * Tensor-memory drain rate (measurement hook, no reference counterpart): one CTA per SM with
 * `warps` warps (4, 8, 12 or 16), each reading its 32-lane quarter `iters` times with `depth`
 * (1, 2 or 4) tcgen05.ld 32x32b.x16 loads in flight before one wait.  *bytes_out receives the
 * bytes the launch moved from tensor memory to registers; the caller times the launch.
 */
int hy3d_probe_tmem_ld(int warps, int depth, int iters, int64_t* bytes_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HY3D_INT8_H_ */
