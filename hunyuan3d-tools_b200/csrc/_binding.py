"""ctypes binding of ``libhy3d_int8.so`` with the reference's extension function names.

The reference exposes three pybind modules (``csrc/int8_gemm_tc.cu:323-328``,
``csrc/int8_sparse_tc.cu:2046-2073``, ``csrc/int8_kernels.cu:213-220``).  The classes below
offer the same callables -- same names, argument order and meaning -- over the C ABI declared
in ``include/hy3d_int8.h``.  Differences, all additive:

* bf16 activations / scales / bias are accepted next to fp16; the output dtype follows x;
* every kernel is launched on the current torch stream;
* errors come back as integer status codes and are raised as ``RuntimeError``.

Outputs and workspaces are allocated here with torch (the C ABI never allocates).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int64, c_void_p

import torch

F16, BF16, F32, S32 = 0, 1, 2, 3
EPI_LINEAR, EPI_GELU, EPI_GEGLU = 0, 1, 2

_DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32, torch.int32: S32}

# name -> (argtypes); every function returns int.  Kept in one table so the CPU test can
# check that the library exports exactly what the header declares.
SIGNATURES = {
    "hy3d_quantize_rows": [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p],
    "hy3d_quantizer_enum_check": [c_int, c_void_p, c_void_p, c_void_p],
    "hy3d_layernorm_quantize": [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int,
                                ctypes.c_float, c_void_p, c_void_p, c_void_p, c_void_p],
    "hy3d_gemm_w8a8_dense": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                             c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int,
                             c_void_p],
    "hy3d_dense_splitk_plan": [c_int64, c_int64, c_int64, c_int, c_void_p],
    "hy3d_gemm_w8a8_dense_splitk": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                    c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p],
    "hy3d_linear_w8a8_dense": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_int, c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64,
                               c_int, c_int, c_int, c_void_p],
    "hy3d_linear_w8a8_dense_fused": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                     c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64,
                                     c_int, c_int, c_void_p],
    "hy3d_linear_path": [c_int64, c_int64, c_int64, c_int],
    "hy3d_linear_w8a8_dense_static": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p,
                                      c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int,
                                      c_void_p],
    "hy3d_prune_pack_24": [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                           c_void_p],
    "hy3d_gemm_w8a8_sparse24": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int,
                                c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64,
                                c_int, c_int, c_void_p],
    "hy3d_linear_w8a8_sparse24": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int64, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                  c_int64, c_int64, c_int64, c_int, c_int, c_void_p],
    "hy3d_dequant_bias": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                          c_int64, c_int64, c_void_p],
    "hy3d_mma_kat": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "hy3d_last_device_status": [c_void_p],
    "hy3d_stream_status": [c_void_p],
    "hy3d_set_wait_limit_ns": [ctypes.c_ulonglong],
    "hy3d_wait_selftest": [c_void_p],
    "hy3d_probe_mma_i8": [c_int, c_int, c_int, c_void_p, c_void_p],
    "hy3d_probe_hbm": [c_int, c_void_p, c_void_p, c_int64, c_void_p],
    "hy3d_probe_tmem_ld": [c_int, c_int, c_int, c_void_p, c_void_p],
    "hy3d_groupnorm_nhwc": [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p,
                            c_int, ctypes.c_float, c_int, c_void_p, c_void_p, c_void_p],
    "hy3d_version": [],
}

# The argument lists above belong to this ABI version of the library (hy3d_version()).
ABI_VERSION = 201


def configure(lib: ctypes.CDLL) -> ctypes.CDLL:
    """Sets argument / result types and refuses a library built for another ABI version: a
    stale .so driven with newer argument lists would hand wrong pointers to the kernels."""
    lib.hy3d_version.argtypes = []
    lib.hy3d_version.restype = c_int
    found = lib.hy3d_version()
    if found != ABI_VERSION:
        raise RuntimeError(f"libhy3d_int8.so has ABI version {found}, this binding needs "
                           f"{ABI_VERSION}; rebuild it with `python csrc/build.py`")
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    for name in ("hy3d_static_scratch_max_bytes", "hy3d_static_scratch_max_rows"):
        getattr(lib, name).restype = c_int64
        getattr(lib, name).argtypes = []
    lib.hy3d_groupnorm_workspace_floats.restype = c_int64
    lib.hy3d_groupnorm_workspace_floats.argtypes = [c_int64, c_int64, c_int]
    lib.hy3d_arch.restype = ctypes.c_char_p
    lib.hy3d_arch.argtypes = []
    lib.hy3d_source_digest.restype = ctypes.c_char_p
    lib.hy3d_source_digest.argtypes = []
    lib.hy3d_status_string.restype = ctypes.c_char_p
    lib.hy3d_status_string.argtypes = [c_int]
    return lib


def meta_words_per_row(K: int) -> int:
    """Row pitch (uint32 words) of the packed 2:4 metadata: K/32 rounded up to whole
    128-deep K blocks, the unit the sparse GEMM loads."""
    return 4 * ((K + 127) // 128)


class _Base:
    def __init__(self, lib: ctypes.CDLL):
        self._lib = configure(lib)

    # -- helpers -----------------------------------------------------------------------
    def _check(self, status: int, what: str):
        if status != 0:
            msg = self._lib.hy3d_status_string(status).decode()
            raise RuntimeError(f"{what} failed: {msg} (status {status})")

    @staticmethod
    def _stream(t: torch.Tensor) -> int:
        return torch.cuda.current_stream(t.device).cuda_stream

    @staticmethod
    def _req(t: torch.Tensor, name: str, dtype=None, dim=None):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
            raise RuntimeError(f"{name} has dtype {t.dtype}, expected {dtype}")
        if dim is not None and t.dim() != dim:
            raise RuntimeError(f"{name} must be {dim}-D")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")

    @staticmethod
    def _opt_bias(bias):
        """The reference passes "no bias" as a zero-element tensor."""
        if bias is None or bias.numel() == 0:
            return None, F16
        return bias.data_ptr(), _DTYPE_CODE[bias.dtype]

    def device_status(self) -> int:
        """Reads and clears the device-side error word (synchronises the device)."""
        v = c_int(0)
        self._check(self._lib.hy3d_last_device_status(ctypes.byref(v)), "hy3d_last_device_status")
        return v.value

    def check_stream(self, device=None):
        """Waits for the current stream and raises if a kernel gave up one of its bounded
        waits (its output is then undefined); the error word is cleared by the raise."""
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        with torch.cuda.device(dev):
            rc = self._lib.hy3d_stream_status(torch.cuda.current_stream(dev).cuda_stream)
            if rc != 0:
                code = self.device_status() if rc == 5 else 0
                msg = self._lib.hy3d_status_string(rc).decode()
                raise RuntimeError(f"{msg} (status {rc}, device code {code})")

    # -- shared kernels ------------------------------------------------------------------
    def _quantize(self, x: torch.Tensor):
        self._req(x, "x", (torch.float16, torch.bfloat16), 2)
        M, K = x.shape
        q = torch.empty((M, K), dtype=torch.int8, device=x.device)
        s = torch.empty((M,), dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            self._check(self._lib.hy3d_quantize_rows(x.data_ptr(), _DTYPE_CODE[x.dtype], M, K, K,
                                                     q.data_ptr(), s.data_ptr(), self._stream(x)),
                        "hy3d_quantize_rows")
        return q, s

    def layernorm_quantize(self, x, gamma, beta, eps, return_normalised=False):
        """LayerNorm over the last dimension of x (M,K) f16/bf16 fused with the per-token
        quantiser: returns (int8 (M,K), f32 scale (M)[, normalised activations (M,K)]) equal to
        quantising the rounded LayerNorm output, without writing that output."""
        self._req(x, "x", (torch.float16, torch.bfloat16), 2)
        M, K = x.shape
        q = torch.empty((M, K), dtype=torch.int8, device=x.device)
        s = torch.empty((M,), dtype=torch.float32, device=x.device)
        y = torch.empty_like(x) if return_normalised else None
        if gamma is not None and beta is not None and gamma.dtype != beta.dtype:
            beta = beta.to(gamma.dtype)
        gb = gamma if gamma is not None else beta
        code = _DTYPE_CODE[gb.dtype] if gb is not None else F32
        with torch.cuda.device(x.device):
            self._check(self._lib.hy3d_layernorm_quantize(
                x.data_ptr(), _DTYPE_CODE[x.dtype], M, K, K,
                gamma.data_ptr() if gamma is not None else None,
                beta.data_ptr() if beta is not None else None, code, float(eps),
                q.data_ptr(), s.data_ptr(), y.data_ptr() if y is not None else None, self._stream(x)),
                "hy3d_layernorm_quantize")
        return (q, s, y) if return_normalised else (q, s)

    def groupnorm_nhwc(self, x, groups, gamma, beta, eps, silu=False, out=None, workspace=None, add=None):
        """GroupNorm (+ SiLU) of a channels_last (B, C, H, W) f16/bf16 tensor; the result has
        the same shape and memory format.  ``workspace``: optional fp32 tensor of at least
        ``groupnorm_workspace_floats(B, H*W, groups)`` elements (allocated when absent).
        ``add``: optional (B, C) tensor of x's dtype added per sample and channel first."""
        if x.dim() != 4 or x.dtype not in (torch.float16, torch.bfloat16) or not x.is_cuda:
            raise RuntimeError("groupnorm_nhwc: x must be a 4-D f16/bf16 CUDA tensor")
        if not x.is_contiguous(memory_format=torch.channels_last):
            raise RuntimeError("groupnorm_nhwc: x must be in channels_last memory format")
        B, C, H, W = x.shape
        if add is not None:
            if tuple(add.shape) != (B, C) or add.dtype != x.dtype or not add.is_cuda:
                raise RuntimeError(f"groupnorm_nhwc: add must be a ({B}, {C}) CUDA tensor of {x.dtype}")
            add = add.contiguous()
        y = out if out is not None else torch.empty_like(x, memory_format=torch.channels_last)
        need = self._lib.hy3d_groupnorm_workspace_floats(B, H * W, groups)
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(max(need, 1), dtype=torch.float32, device=x.device)
        if gamma is not None and beta is not None and gamma.dtype != beta.dtype:
            beta = beta.to(gamma.dtype)
        gb = gamma if gamma is not None else beta
        code = _DTYPE_CODE[gb.dtype] if gb is not None else F32
        with torch.cuda.device(x.device):
            self._check(self._lib.hy3d_groupnorm_nhwc(
                x.data_ptr(), add.data_ptr() if add is not None else None, _DTYPE_CODE[x.dtype], B, H * W, C, groups,
                gamma.data_ptr() if gamma is not None else None,
                beta.data_ptr() if beta is not None else None, code, float(eps), 1 if silu else 0,
                y.data_ptr(), workspace.data_ptr(), self._stream(x)), "hy3d_groupnorm_nhwc")
        return y

    def quantizer_enum_check(self, dtype):
        """(pairs checked, codes differing from rint(x / scale)) over every 16-bit (amax, x)."""
        pairs, bad = ctypes.c_ulonglong(0), ctypes.c_ulonglong(0)
        self._check(self._lib.hy3d_quantizer_enum_check(
            _DTYPE_CODE[dtype], ctypes.byref(pairs), ctypes.byref(bad),
            torch.cuda.current_stream().cuda_stream), "hy3d_quantizer_enum_check")
        return pairs.value, bad.value

    def _out_shape(self, M, N, epilogue):
        return (M, N // 2) if epilogue == EPI_GEGLU else (M, N)


class Int8KernelsModule(_Base):
    """Counterpart of the reference's ``int8_kernels`` extension (csrc/int8_kernels.cu)."""

    def fused_quantize_activation(self, x):
        """x (M,K) f16/bf16 -> (int8 (M,K), f32 scale (M)).  csrc/int8_kernels.cu:128-153."""
        return self._quantize(x)

    def fused_dequantize_bias(self, acc, act_scale, w_scale, bias, out_dtype=None):
        """int32 (M,N) -> (M,N) f16/bf16.  csrc/int8_kernels.cu:156-190."""
        self._req(acc, "acc", torch.int32, 2)
        self._req(act_scale, "act_scale", torch.float32, 1)
        self._req(w_scale, "w_scale", (torch.float16, torch.bfloat16, torch.float32), 1)
        M, N = acc.shape
        if out_dtype is None:
            out_dtype = w_scale.dtype if w_scale.dtype != torch.float32 else torch.float16
        out = torch.empty((M, N), dtype=out_dtype, device=acc.device)
        bptr, bcode = self._opt_bias(bias)
        with torch.cuda.device(acc.device):
            self._check(self._lib.hy3d_dequant_bias(acc.data_ptr(), act_scale.data_ptr(),
                                                    w_scale.data_ptr(), _DTYPE_CODE[w_scale.dtype],
                                                    bptr, bcode, out.data_ptr(),
                                                    _DTYPE_CODE[out_dtype], M, N, self._stream(acc)),
                        "hy3d_dequant_bias")
        return out

    def int8_linear_fused(self, x, w_int8_t, w_scale, bias):
        """x (M,K) f16/bf16, w_int8_t (K,N) int8 -> (M,N).  csrc/int8_kernels.cu:193-210.
        The reference ran quantise -> torch::_int_mm -> dequant; here the (K,N) weight is
        viewed back as (N,K) and the fused tensor-core path runs."""
        w_nk = w_int8_t.t().contiguous()
        return TcGemmModule(self._lib).int8_linear_tc(x, w_nk, w_scale, bias)


class TcGemmModule(_Base):
    """Counterpart of the reference's ``int8_gemm_tc`` extension (csrc/int8_gemm_tc.cu)."""

    def dense_splitk_plan(self, M, N, K, epilogue=EPI_LINEAR):
        """(K ranges this library would use for the shape -- 1 = no split --, workspace bytes)."""
        nbytes = ctypes.c_int64(0)
        splits = self._lib.hy3d_dense_splitk_plan(M, N, K, epilogue, ctypes.byref(nbytes))
        return int(splits), int(nbytes.value)

    def int8_gemm_tc(self, A, B, act_scale, w_scale, bias, out_dtype=None, epilogue=EPI_LINEAR,
                     cta_group=0, block_n=0, splits=None):
        """A (M,K) s8, B (N,K) s8, act_scale (M) f32, w_scale (N), bias (N) or empty ->
        (M,N).  csrc/int8_gemm_tc.cu:254-309.  ``out_dtype=torch.int32`` returns the raw
        accumulators.  ``splits``: K ranges of the split-K form (None = the library's plan for
        the shape, 1 = never split); the result is the same bit for bit."""
        self._req(A, "A", torch.int8, 2)
        self._req(B, "B", torch.int8, 2)
        M, K = A.shape
        N, K2 = B.shape
        if K != K2:
            raise RuntimeError(f"K mismatch: A has {K}, B has {K2}")
        if out_dtype is None:
            out_dtype = w_scale.dtype if w_scale.dtype != torch.float32 else torch.float16
        out = torch.empty(self._out_shape(M, N, epilogue), dtype=out_dtype, device=A.device)
        bptr, bcode = self._opt_bias(bias)
        if splits is None:
            splits = self.dense_splitk_plan(M, N, K, epilogue)[0] if (
                out_dtype in (torch.float16, torch.bfloat16) and cta_group == 0 and block_n == 0) else 1
        if splits > 1:
            ws = torch.empty((splits, (M + 127) // 128 * 128, N), dtype=torch.int32, device=A.device)
            with torch.cuda.device(A.device):
                self._check(self._lib.hy3d_gemm_w8a8_dense_splitk(
                    A.data_ptr(), B.data_ptr(), act_scale.data_ptr(), w_scale.data_ptr(),
                    _DTYPE_CODE[w_scale.dtype], bptr, bcode, out.data_ptr(), _DTYPE_CODE[out_dtype],
                    M, N, K, epilogue, splits, ws.data_ptr(), ws.numel() * 4, self._stream(A)),
                    "hy3d_gemm_w8a8_dense_splitk")
            return out
        as_ptr = act_scale.data_ptr() if act_scale is not None else None
        ws_ptr = w_scale.data_ptr() if w_scale is not None else None
        ws_code = _DTYPE_CODE[w_scale.dtype] if w_scale is not None else F32
        with torch.cuda.device(A.device):
            self._check(self._lib.hy3d_gemm_w8a8_dense(
                A.data_ptr(), B.data_ptr(), as_ptr, ws_ptr, ws_code, bptr, bcode, out.data_ptr(),
                _DTYPE_CODE[out_dtype], M, N, K, epilogue, cta_group, block_n, self._stream(A)),
                "hy3d_gemm_w8a8_dense")
        return out

    def int8_linear_tc_fused(self, x, w_int8, w_scale, bias, epilogue=EPI_LINEAR, block_n=0,
                             return_scales=False):
        """``int8_linear_tc`` as one launch with the quantised activations resident in shared
        memory (the role of the reference's fused path, csrc/int8_sparse_tc.cu:1934-2002).
        Bit-identical to the two-launch path; raises for shapes the kernel does not take
        (K > 1280, K % 32 != 0)."""
        self._req(x, "x", (torch.float16, torch.bfloat16), 2)
        self._req(w_int8, "w_int8", torch.int8, 2)
        M, K = x.shape
        N = w_int8.shape[0]
        if w_int8.shape[1] != K:
            raise RuntimeError(f"K mismatch: x has {K}, w_int8 has {w_int8.shape[1]}")
        out = torch.empty(self._out_shape(M, N, epilogue), dtype=x.dtype, device=x.device)
        s = torch.empty((M,), dtype=torch.float32, device=x.device) if return_scales else None
        bptr, bcode = self._opt_bias(bias)
        with torch.cuda.device(x.device):
            self._check(self._lib.hy3d_linear_w8a8_dense_fused(
                x.data_ptr(), _DTYPE_CODE[x.dtype], K, s.data_ptr() if s is not None else None,
                w_int8.data_ptr(), w_scale.data_ptr(), _DTYPE_CODE[w_scale.dtype], bptr, bcode,
                out.data_ptr(), _DTYPE_CODE[x.dtype], M, N, K, epilogue, block_n,
                self._stream(x)), "hy3d_linear_w8a8_dense_fused")
        return (out, s) if return_scales else out

    def int8_linear_path(self, M, K, N, epilogue=EPI_LINEAR):
        """1 when ``int8_linear_tc`` runs this shape as one launch, 0 for two (the dense
        counterpart of csrc/int8_sparse_tc.cu:2065-2070)."""
        return int(self._lib.hy3d_linear_path(M, K, N, epilogue))

    def int8_linear_tc(self, x, w_int8, w_scale, bias, epilogue=EPI_LINEAR, cta_group=0, block_n=0):
        """x (M,K) f16/bf16, w_int8 (N,K), w_scale (N), bias (N) or empty -> (M,N) in x's
        dtype.  csrc/int8_gemm_tc.cu:312-320."""
        self._req(x, "x", (torch.float16, torch.bfloat16), 2)
        self._req(w_int8, "w_int8", torch.int8, 2)
        M, K = x.shape
        N = w_int8.shape[0]
        if w_int8.shape[1] != K:
            raise RuntimeError(f"K mismatch: x has {K}, w_int8 has {w_int8.shape[1]}")
        if cta_group == 0 and block_n == 0 and self.dense_splitk_plan(M, N, K, epilogue)[0] > 1:
            q, s = self._quantize(x)                     # few rows, deep K: split-K GEMM
            return self.int8_gemm_tc(q, w_int8, s, w_scale, bias, out_dtype=x.dtype, epilogue=epilogue)
        q = torch.empty((M, K), dtype=torch.int8, device=x.device)
        s = torch.empty((M,), dtype=torch.float32, device=x.device)
        out = torch.empty(self._out_shape(M, N, epilogue), dtype=x.dtype, device=x.device)
        bptr, bcode = self._opt_bias(bias)
        with torch.cuda.device(x.device):
            self._check(self._lib.hy3d_linear_w8a8_dense(
                x.data_ptr(), _DTYPE_CODE[x.dtype], K, q.data_ptr(), s.data_ptr(),
                w_int8.data_ptr(), w_scale.data_ptr(), _DTYPE_CODE[w_scale.dtype], bptr, bcode,
                out.data_ptr(), _DTYPE_CODE[x.dtype], M, N, K, epilogue, cta_group, block_n,
                self._stream(x)), "hy3d_linear_w8a8_dense")
        return out

    def int8_linear_tc_static(self, x, w_int8, w_scale, bias, out=None, epilogue=EPI_LINEAR):
        """``int8_linear_tc`` through the entry point that keeps its scratch inside the
        library, for callers that cannot allocate where the layer runs.  Pass ``out`` to make
        the call itself allocation-free; M*K and M are limited (see the header)."""
        self._req(x, "x", (torch.float16, torch.bfloat16), 2)
        self._req(w_int8, "w_int8", torch.int8, 2)
        M, K = x.shape
        N = w_int8.shape[0]
        if w_int8.shape[1] != K:
            raise RuntimeError(f"K mismatch: x has {K}, w_int8 has {w_int8.shape[1]}")
        if out is None:
            out = torch.empty(self._out_shape(M, N, epilogue), dtype=x.dtype, device=x.device)
        bptr, bcode = self._opt_bias(bias)
        with torch.cuda.device(x.device):
            self._check(self._lib.hy3d_linear_w8a8_dense_static(
                x.data_ptr(), _DTYPE_CODE[x.dtype], K, w_int8.data_ptr(), w_scale.data_ptr(),
                _DTYPE_CODE[w_scale.dtype], bptr, bcode, out.data_ptr(), _DTYPE_CODE[out.dtype],
                M, N, K, epilogue, self._stream(x)), "hy3d_linear_w8a8_dense_static")
        return out

    def test_mma(self, a, b):
        """One dense tensor-core tile: a (128,k) s8, b (n,k) s8 -> (128,n) int32, k = 32..128."""
        self._req(a, "a", torch.int8, 2)
        self._req(b, "b", torch.int8, 2)
        n, k = b.shape
        d = torch.empty((128, n), dtype=torch.int32, device=a.device)
        with torch.cuda.device(a.device):
            self._check(self._lib.hy3d_mma_kat(a.data_ptr(), b.data_ptr(), None, d.data_ptr(), n,
                                               k // 32, 0, self._stream(a)), "hy3d_mma_kat")
        return d


class SparseTcModule(_Base):
    """Counterpart of the reference's ``int8_sparse_tc`` extension (csrc/int8_sparse_tc.cu)."""

    def sparse_prune_compress(self, w):
        """w (N,K) s8 -> (comp (N,K/2) s8, meta_raw (N*K/4) u8, one nibble per byte).
        csrc/int8_sparse_tc.cu:1558-1585."""
        self._req(w, "w", torch.int8, 2)
        N, K = w.shape
        comp = torch.empty((N, K // 2), dtype=torch.int8, device=w.device)
        raw = torch.empty((N * K // 4,), dtype=torch.uint8, device=w.device)
        with torch.cuda.device(w.device):
            self._check(self._lib.hy3d_prune_pack_24(w.data_ptr(), N, K, comp.data_ptr(),
                                                     raw.data_ptr(), None, 0, self._stream(w)),
                        "hy3d_prune_pack_24")
        return comp, raw

    def sparse_prune_and_pack(self, w):
        """w (N,K) s8 -> (comp (N,K/2) s8, meta (N, 4*ceil(K/128)) int32).  The metadata
        words hold 8 nibbles each, least-significant first, as in the reference
        (csrc/int8_sparse_tc.cu:416-437, 1616-1665); rows are padded to whole 128-deep K
        blocks, so the shape equals the reference's (N, K/32) whenever K % 128 == 0."""
        self._req(w, "w", torch.int8, 2)
        N, K = w.shape
        ld = meta_words_per_row(K)
        comp = torch.empty((N, K // 2), dtype=torch.int8, device=w.device)
        meta = torch.empty((N, ld), dtype=torch.int32, device=w.device)
        with torch.cuda.device(w.device):
            self._check(self._lib.hy3d_prune_pack_24(w.data_ptr(), N, K, comp.data_ptr(), None,
                                                     meta.data_ptr(), ld, self._stream(w)),
                        "hy3d_prune_pack_24")
        return comp, meta

    def sparse_quantize_act(self, x):
        """csrc/int8_sparse_tc.cu:1668-1707."""
        return self._quantize(x)

    def sparse_int8_gemm(self, x_int8, act_scale, w_comp, w_meta, w_scale, bias, force_tile=-1,
                         force_split=-1, force_order=-1, out_dtype=None, epilogue=EPI_LINEAR):
        """csrc/int8_sparse_tc.cu:1758-1929.  ``force_tile`` > 0 sets the token-tile width;
        ``force_split`` / ``force_order`` are accepted for signature compatibility (there is
        no split-K: accumulation is int32 throughout)."""
        self._req(x_int8, "x_int8", torch.int8, 2)
        self._req(w_comp, "w_comp", torch.int8, 2)
        self._req(w_meta, "w_meta", torch.int32, 2)
        M, K = x_int8.shape
        N = w_comp.shape[0]
        if w_comp.shape[1] * 2 != K:
            raise RuntimeError("w_comp must be (N, K/2)")
        if out_dtype is None:
            out_dtype = w_scale.dtype if w_scale.dtype != torch.float32 else torch.float16
        out = torch.empty(self._out_shape(M, N, epilogue), dtype=out_dtype, device=x_int8.device)
        bptr, bcode = self._opt_bias(bias)
        as_ptr = act_scale.data_ptr() if act_scale is not None else None
        ws_ptr = w_scale.data_ptr() if w_scale is not None else None
        ws_code = _DTYPE_CODE[w_scale.dtype] if w_scale is not None else F32
        with torch.cuda.device(x_int8.device):
            self._check(self._lib.hy3d_gemm_w8a8_sparse24(
                x_int8.data_ptr(), as_ptr, w_comp.data_ptr(), w_meta.data_ptr(), w_meta.shape[1],
                ws_ptr, ws_code, bptr, bcode, out.data_ptr(), _DTYPE_CODE[out_dtype], M, N, K,
                epilogue, max(force_tile, 0), self._stream(x_int8)), "hy3d_gemm_w8a8_sparse24")
        return out

    def sparse_int8_linear_ex(self, x, w_comp, w_meta, w_scale, bias, path=-1, epilogue=EPI_LINEAR):
        """csrc/int8_sparse_tc.cu:2006-2025.  ``path`` is accepted and ignored."""
        self._req(x, "x", (torch.float16, torch.bfloat16), 2)
        self._req(w_comp, "w_comp", torch.int8, 2)
        self._req(w_meta, "w_meta", torch.int32, 2)
        M, K = x.shape
        N = w_comp.shape[0]
        if w_comp.shape[1] * 2 != K:
            raise RuntimeError("w_comp must be (N, K/2)")
        q = torch.empty((M, K), dtype=torch.int8, device=x.device)
        s = torch.empty((M,), dtype=torch.float32, device=x.device)
        out = torch.empty(self._out_shape(M, N, epilogue), dtype=x.dtype, device=x.device)
        bptr, bcode = self._opt_bias(bias)
        with torch.cuda.device(x.device):
            self._check(self._lib.hy3d_linear_w8a8_sparse24(
                x.data_ptr(), _DTYPE_CODE[x.dtype], K, q.data_ptr(), s.data_ptr(),
                w_comp.data_ptr(), w_meta.data_ptr(), w_meta.shape[1], w_scale.data_ptr(),
                _DTYPE_CODE[w_scale.dtype], bptr, bcode, out.data_ptr(), _DTYPE_CODE[x.dtype],
                M, N, K, epilogue, 0, self._stream(x)), "hy3d_linear_w8a8_sparse24")
        return out

    def sparse_int8_linear(self, x, w_comp, w_meta, w_scale, bias):
        """csrc/int8_sparse_tc.cu:2027-2044."""
        return self.sparse_int8_linear_ex(x, w_comp, w_meta, w_scale, bias, -1)

    def sparse_int8_linear_path(self, M, K, N):
        """csrc/int8_sparse_tc.cu:2065-2070 reported which of two code paths a shape takes
        (1 = quantiser fused into the GEMM).  The sparse layer here always runs its
        quantiser and its GEMM as two launches."""
        return 0

    def test_mma_sp(self, a_comp, b, meta):
        """One sparse tensor-core tile: a_comp (128,k/2) s8, b (n,k) s8, meta (128,4) int32
        -> D (128,n) int32 with D = expand(a_comp, meta) @ b^T; k = 64 or 128.
        Stands in for csrc/int8_sparse_tc.cu:1587-1614 (test_mma_sp)."""
        self._req(a_comp, "a_comp", torch.int8, 2)
        self._req(b, "b", torch.int8, 2)
        self._req(meta, "meta", torch.int32, 2)
        n, k = b.shape
        dt = torch.empty((n, 128), dtype=torch.int32, device=b.device)
        with torch.cuda.device(b.device):
            self._check(self._lib.hy3d_mma_kat(a_comp.data_ptr(), b.data_ptr(), meta.data_ptr(),
                                               dt.data_ptr(), n, k // 64, 1, self._stream(b)),
                        "hy3d_mma_kat")
        return dt.t().contiguous()
