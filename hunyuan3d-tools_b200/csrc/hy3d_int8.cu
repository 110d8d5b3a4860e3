// Single translation unit of libhy3d_int8.so: the kernel files are included here so that
// they share one copy of the device-side status word without relocatable device code.
#include "quantize.cu"
#include "prune_pack.cu"
#include "gemm_dense.cu"
#include "gemm_sparse.cu"
#include "linear_fused.cu"
#include "groupnorm.cu"
#include "capi.cu"
#include "static_scratch.cu"
#include "probes.cu"
