"""INT8 linear layers for the Hunyuan3D-2.1 texture UNet on B200 (sm_100a).

Drop-in for the reference's ``quantize_utils.py``: the same public names
(``Int8Linear``, ``quantize_model_tensorcore``, ``quantize_model_sparse``, ``tc_available``,
``sp_available``), the same buffers (``weight_int8_nk``, ``weight_scale``,
``weight_sparse_comp``, ``weight_sparse_meta``, ``bias``), the same per-output-channel weight
scales, per-token activation scales and stats dictionaries (reference
``quantize_utils.py:151-498``).

Compute backends:

* ``"tc"``     dense W8A8: fused per-token quantise kernel + ``tcgen05.mma kind::i8`` GEMM
               with the rescale / bias (/ GELU / GEGLU) epilogue.
* ``"sparse"`` 2:4 structured-sparse W8A8 on ``tcgen05.mma.sp``.

There is deliberately no CPU, Triton, ``torch._int_mm`` or dequantise fallback here: if the
CUDA library cannot be loaded, or the input is not on a CUDA device, the layer raises.  The
reference's fallbacks (``_forward_int_mm``, ``_forward_dequant``, quantize_utils.py:293-314)
exist in this repository only inside the test oracle.

Differences from the reference, all of them additive:

* activations, scales and bias may be bf16 as well as fp16; scale and bias buffers take the
  dtype of the source ``nn.Linear`` (fp32 sources are stored as fp16, as in the reference);
* the tensor-core path handles any M >= 1 (the reference fell back below 256 rows,
  quantize_utils.py:324, 336);
* ``Int8Linear.epilogue`` selects a fused activation ("linear", "gelu", "geglu");
* sparse metadata rows are padded to whole 128-deep K blocks: shape (N, 4*ceil(K/128)),
  equal to the reference's (N, K/32) whenever K % 128 == 0.
"""
from __future__ import annotations

import os

import torch
import torch.nn as nn

# Same switch as the reference (quantize_utils.py:43-44).  A load failure is always an
# error here; the variable is read so that scripts which set it keep working.
_STRICT = os.environ.get("INT8_KERNELS_STRICT", "") not in ("", "0")
_FAILED = object()

_EPILOGUES = {"linear": 0, "gelu": 1, "geglu": 2}


def _kernel_unavailable(name, err):
    msg = (f"{name} kernel library failed to build or load: {type(err).__name__}: {err}. "
           "This package has no fallback path; build it with `python csrc/build.py`.")
    raise RuntimeError(msg) from err


# ---------------------------------------------------------------------------------------
#  Lazy extension loading (reference: quantize_utils.py:65-116)
# ---------------------------------------------------------------------------------------
_TC_MODULE = None
_SP_MODULE = None


def _load_tc():
    """Lazy-load the dense tensor-core GEMM module."""
    global _TC_MODULE
    if _TC_MODULE is None:
        try:
            from .csrc.build import load_tc_gemm
            _TC_MODULE = load_tc_gemm()
        except Exception as e:  # noqa: BLE001 - reported with its type, then re-raised
            _kernel_unavailable("Dense INT8 tensor-core GEMM", e)
    return _TC_MODULE


def tc_available() -> bool:
    """True when the dense kernel library loads (raises, as STRICT does, when it cannot)."""
    return _load_tc() is not None


def _load_sp():
    """Lazy-load the 2:4 sparse tensor-core GEMM module."""
    global _SP_MODULE
    if _SP_MODULE is None:
        try:
            from .csrc.build import load_sparse_tc
            _SP_MODULE = load_sparse_tc()
        except Exception as e:  # noqa: BLE001
            _kernel_unavailable("Sparse INT8 tensor-core GEMM", e)
    return _SP_MODULE


def sp_available() -> bool:
    return _load_sp() is not None


def _param_dtype(linear: nn.Linear) -> torch.dtype:
    dt = linear.weight.dtype
    return dt if dt in (torch.float16, torch.bfloat16) else torch.float16


# ---------------------------------------------------------------------------------------
#  Activations that arrive already quantised (emitted by the producing op)
# ---------------------------------------------------------------------------------------
class QuantizedActivation:
    """Per-token int8 codes and scales of an activation tensor, as ``Int8LayerNorm`` emits
    them, with the logical shape and dtype the unquantised tensor would have had.  An
    ``Int8Linear`` given one of these skips its own quantise pass and runs the GEMM directly;
    several sibling layers (q / k / v, the multiview projections, the FFN up-projection) can
    consume the same object."""

    __slots__ = ("q", "scale", "shape", "dtype")

    def __init__(self, q, scale, shape, dtype):
        self.q, self.scale, self.shape, self.dtype = q, scale, torch.Size(shape), dtype

    @property
    def device(self):
        return self.q.device

    @property
    def is_cuda(self):
        return self.q.is_cuda

    def dim(self):
        return len(self.shape)

    def view(self, *shape):
        """Re-labels the leading dimensions (tokens stay tokens: the last dimension is fixed)."""
        shape = tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)) else shape
        probe = torch.empty(self.shape, device="meta").view(*shape)
        if probe.shape[-1] != self.shape[-1]:
            raise RuntimeError("a quantised activation can only be reshaped over its token dimensions")
        return QuantizedActivation(self.q, self.scale, probe.shape, self.dtype)

    reshape = view


class Int8LayerNorm(nn.Module):
    """``nn.LayerNorm`` over the last dimension whose output is emitted as int8 codes plus
    per-token scales (``QuantizedActivation``) by one kernel, so the normalised activations
    are never written and the consuming ``Int8Linear`` layers do not quantise again.  The codes
    equal those the consumers would have computed from the rounded LayerNorm output.  Only for
    LayerNorms whose every consumer is an ``Int8Linear`` (see ``unet.fuse_layernorm_quant``)."""

    def __init__(self, norm: nn.LayerNorm):
        super().__init__()
        if len(norm.normalized_shape) != 1:
            raise RuntimeError("Int8LayerNorm normalises the last dimension only")
        self.normalized_shape = norm.normalized_shape
        self.eps = norm.eps
        self.weight = norm.weight
        self.bias = norm.bias
        self._ik = None

    def forward(self, x: torch.Tensor) -> QuantizedActivation:
        if not x.is_cuda:
            raise RuntimeError("Int8LayerNorm runs on CUDA tensors only (no CPU fallback)")
        if self._ik is None:
            from .csrc.build import load_int8_kernels
            self._ik = load_int8_kernels()
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        q, s = self._ik.layernorm_quantize(x2, self.weight, self.bias, self.eps)
        return QuantizedActivation(q, s, x.shape, x.dtype)

    def extra_repr(self) -> str:
        return f"{self.normalized_shape}, eps={self.eps}, output=int8 codes + per-token scales"


# ---------------------------------------------------------------------------------------
#  Int8Linear
# ---------------------------------------------------------------------------------------
class Int8Linear(nn.Module):
    """Drop-in ``nn.Linear`` replacement with int8 weights (reference: quantize_utils.py:151-371).

    Weight quantisation (offline, per output channel)::

        scale_j     = max(|W[j,:]|) / 127
        W_int8[j,:] = round(W[j,:] / scale_j).clamp(-128, 127)
    """

    __constants__ = ["in_features", "out_features", "_tc_ok", "_sparse_ok"]

    # "tc" (dense) or "sparse"; a plain attribute, set per instance by from_linear_sparse.
    mode: str = "tc"
    # "linear", "gelu" or "geglu" (GEGLU halves the output width and expects the weight rows
    # interleaved by ``interleave_geglu_rows``).
    epilogue: str = "linear"

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 dtype: torch.dtype = torch.float16):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        # The reference's eligibility rule (quantize_utils.py:175-178).
        self._tc_ok = (in_features % 64 == 0) and (out_features % 16 == 0)
        self._sparse_ok = (in_features % 64 == 0) and (out_features % 16 == 0)
        self.register_buffer("weight_int8_nk", torch.zeros(out_features, in_features, dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_features, dtype=dtype))
        self.register_buffer("weight_sparse_comp", None)
        self.register_buffer("weight_sparse_meta", None)
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=dtype))
        else:
            self.bias = None

    # -- construction ------------------------------------------------------------------
    @staticmethod
    def from_linear(linear: nn.Linear) -> "Int8Linear":
        """Per-channel quantisation of an ``nn.Linear`` (reference: quantize_utils.py:203-223)."""
        has_bias = linear.bias is not None
        dt = _param_dtype(linear)
        layer = Int8Linear(linear.in_features, linear.out_features, bias=has_bias, dtype=dt)
        weight_f32 = linear.weight.data.float()
        # Same expressions as the reference, evaluated on the weight's device.  (On CUDA torch
        # divides by a Python scalar through its reciprocal, so a scale can differ by one ulp
        # from the CPU value; the reference behaves the same way.)
        scale = weight_f32.abs().amax(dim=1) / 127.0
        scale = scale.clamp(min=1e-8)
        weight_int8 = (weight_f32 / scale[:, None]).round().clamp(-128, 127).to(torch.int8)
        layer.weight_int8_nk = weight_int8.contiguous()
        layer.weight_scale = scale.to(dt)
        if has_bias:
            layer.bias = linear.bias.data.to(dt)
        return layer.to(linear.weight.device)

    @staticmethod
    def from_linear_sparse(linear: nn.Linear) -> "Int8Linear":
        """2:4-sparse conversion (reference: quantize_utils.py:226-260): quantise with the
        scale of the UNPRUNED row, then prune on int8 magnitudes, compress and pack on the
        GPU."""
        sp_mod = _load_sp()
        has_bias = linear.bias is not None
        dt = _param_dtype(linear)
        device = linear.weight.device
        if device.type != "cuda":
            raise RuntimeError("from_linear_sparse needs the layer on a CUDA device "
                               "(pruning and packing run on the GPU)")
        layer = Int8Linear(linear.in_features, linear.out_features, bias=has_bias, dtype=dt)
        weight_f32 = linear.weight.data.float()
        scale = weight_f32.abs().amax(dim=1).clamp(min=1e-8) / 127.0
        weight_int8 = (weight_f32 / scale[:, None]).round().clamp(-128, 127).to(torch.int8)
        comp, meta = sp_mod.sparse_prune_and_pack(weight_int8.contiguous())
        layer.weight_sparse_comp = comp
        layer.weight_sparse_meta = meta
        layer.weight_scale = scale.to(dt)
        layer.register_buffer("weight_int8_nk", torch.empty(0, dtype=torch.int8))
        if has_bias:
            layer.bias = linear.bias.data.to(dt)
        layer.mode = "sparse"
        return layer.to(device)

    # -- checkpointing -----------------------------------------------------------------
    # The reference registers the sparse buffers as None, so a freshly constructed layer
    # cannot load a sparse checkpoint (quantize_utils.py:190-192).  Here the mode, epilogue
    # and buffer shapes travel with the state dict, so a pruned + packed model reloads
    # without re-pruning.
    def get_extra_state(self):
        return {"mode": self.mode, "epilogue": self.epilogue, "layout": "hy3d-int8-v1"}

    def set_extra_state(self, state):
        self.mode = state.get("mode", "tc")
        self.epilogue = state.get("epilogue", "linear")

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        # Re-shape this layer's buffers to whatever the checkpoint holds (dense weights may be
        # empty, sparse buffers may be present) before the generic copy runs.
        for name in ("weight_int8_nk", "weight_scale", "weight_sparse_comp", "weight_sparse_meta", "bias"):
            key = prefix + name
            if key in state_dict:
                src = state_dict[key]
                cur = getattr(self, name, None)
                if cur is None or cur.shape != src.shape or cur.dtype != src.dtype:
                    device = self.weight_scale.device
                    if name == "bias" and name not in self._buffers:
                        # built with bias=False: the plain None attribute must make room
                        del self.bias
                    self.register_buffer(name, torch.empty(src.shape, dtype=src.dtype, device=device))
        # A checkpoint in the reference's layout (buffers only, quantize_utils.py:181-198) has
        # no extra state: infer it from which buffers are filled.
        if prefix + "_extra_state" not in state_dict:
            comp = state_dict.get(prefix + "weight_sparse_comp")
            dense = state_dict.get(prefix + "weight_int8_nk")
            sparse = comp is not None and comp.numel() > 0 and (dense is None or dense.numel() == 0)
            state_dict[prefix + "_extra_state"] = {"mode": "sparse" if sparse else "tc",
                                                   "epilogue": "linear", "layout": "hy3d-int8-v1"}
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)

    @staticmethod
    def concat(layers) -> "Int8Linear":
        """One layer computing ``[l0(x) | l1(x) | ...]`` for already converted layers that read
        the same input (q/k/v projections): the per-row weight codes, scales, 2:4 metadata and
        biases are stacked along the output dimension, so every output column keeps the bits
        the separate layer would have produced while the activation is quantised once."""
        layers = list(layers)
        first = layers[0]
        for l in layers:
            if not isinstance(l, Int8Linear):
                raise TypeError("Int8Linear.concat takes Int8Linear layers")
            if (l.in_features != first.in_features or l.mode != first.mode or l.epilogue != "linear"
                    or (l.bias is None) != (first.bias is None)
                    or l.weight_scale.dtype != first.weight_scale.dtype):
                raise RuntimeError("Int8Linear.concat needs layers of the same in_features, mode, "
                                   "dtype and bias presence with the plain linear epilogue")
        n = sum(l.out_features for l in layers)
        out = Int8Linear(first.in_features, n, bias=first.bias is not None, dtype=first.weight_scale.dtype)
        out.weight_scale = torch.cat([l.weight_scale for l in layers]).contiguous()
        if first.bias is not None:
            out.bias = torch.cat([l.bias for l in layers]).contiguous()
        if first.mode == "sparse":
            out.weight_sparse_comp = torch.cat([l.weight_sparse_comp for l in layers]).contiguous()
            out.weight_sparse_meta = torch.cat([l.weight_sparse_meta for l in layers]).contiguous()
            out.register_buffer("weight_int8_nk", torch.empty(0, dtype=torch.int8,
                                                              device=first.weight_scale.device))
        else:
            out.weight_int8_nk = torch.cat([l.weight_int8_nk for l in layers]).contiguous()
        out.mode = first.mode
        return out

    def interleave_geglu_rows(self) -> "Int8Linear":
        """Re-orders a GEGLU up-projection ([value(H) | gate(H)] output rows) into blocks of
        16 value rows followed by their 16 gate rows and switches the layer to the fused
        ``value * gelu(gate)`` epilogue; the layer then returns H columns.  Works for dense and
        2:4-sparse layers alike: pruning acts along K inside a row, so permuting whole rows of
        the compressed weights and their metadata commutes with it."""
        if self.mode not in ("tc", "sparse"):
            raise RuntimeError("interleave_geglu_rows applies to INT8 layers")
        if self.epilogue != "linear":
            raise RuntimeError("the layer already has a fused epilogue")
        n2 = self.out_features
        if n2 % 32:
            raise RuntimeError("GEGLU fusion needs out_features % 32 == 0")
        h = n2 // 2
        idx = torch.arange(h, device=self.weight_scale.device).view(h // 16, 16)
        perm = torch.stack([idx, idx + h], dim=1).reshape(-1)
        if self.mode == "sparse":
            self.weight_sparse_comp = self.weight_sparse_comp[perm].contiguous()
            self.weight_sparse_meta = self.weight_sparse_meta[perm].contiguous()
        else:
            self.weight_int8_nk = self.weight_int8_nk[perm].contiguous()
        self.weight_scale = self.weight_scale[perm].contiguous()
        if self.bias is not None:
            self.bias = self.bias[perm].contiguous()
        self.epilogue = "geglu"
        return self

    # -- forward ------------------------------------------------------------------------
    _tc_ref = None
    _sp_ref = None
    _empty_bias = None

    def _bias_or_empty(self, x: torch.Tensor) -> torch.Tensor:
        """"No bias" crosses the extension boundary as a zero-element tensor
        (reference: quantize_utils.py:270-275)."""
        if self.bias is not None:
            return self.bias
        if self._empty_bias is None or self._empty_bias.device != x.device:
            self._empty_bias = torch.empty(0, dtype=x.dtype, device=x.device)
        return self._empty_bias

    def _forward_sparse(self, x: torch.Tensor) -> torch.Tensor:
        if self._sp_ref is None:
            self._sp_ref = _load_sp()
        return self._sp_ref.sparse_int8_linear_ex(
            x, self.weight_sparse_comp, self.weight_sparse_meta, self.weight_scale,
            self._bias_or_empty(x), -1, _EPILOGUES[self.epilogue])

    def _forward_tc(self, x: torch.Tensor) -> torch.Tensor:
        if self._tc_ref is None:
            self._tc_ref = _load_tc()
        return self._tc_ref.int8_linear_tc(x, self.weight_int8_nk, self.weight_scale,
                                           self._bias_or_empty(x), _EPILOGUES[self.epilogue])

    def _forward_quantized(self, x: "QuantizedActivation") -> torch.Tensor:
        """GEMM + epilogue on an activation that was quantised by its producer."""
        epi = _EPILOGUES[self.epilogue]
        if self.mode == "sparse":
            if self._sp_ref is None:
                self._sp_ref = _load_sp()
            y = self._sp_ref.sparse_int8_gemm(x.q, x.scale, self.weight_sparse_comp, self.weight_sparse_meta,
                                              self.weight_scale, self._bias_or_empty(x.q), out_dtype=x.dtype,
                                              epilogue=epi)
        else:
            if self._tc_ref is None:
                self._tc_ref = _load_tc()
            y = self._tc_ref.int8_gemm_tc(x.q, self.weight_int8_nk, x.scale, self.weight_scale,
                                          self._bias_or_empty(x.q), out_dtype=x.dtype, epilogue=epi)
        return y.reshape(*x.shape[:-1], y.shape[-1])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if isinstance(x, QuantizedActivation):
            return self._forward_quantized(x)
        if not x.is_cuda:
            raise RuntimeError("Int8Linear runs on CUDA tensors only (no CPU fallback)")
        if x.dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError(f"Int8Linear expects fp16 or bf16 activations, got {x.dtype}")
        orig_shape = x.shape
        x2 = x.reshape(-1, orig_shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if self.mode == "sparse":
            if not self._sparse_ok:
                raise RuntimeError("sparse Int8Linear needs in_features % 64 == 0 and "
                                   "out_features % 16 == 0")
            y = self._forward_sparse(x2)
        elif self.mode == "tc":
            if not self._tc_ok:
                raise RuntimeError("Int8Linear needs in_features % 64 == 0 and "
                                   "out_features % 16 == 0")
            y = self._forward_tc(x2)
        else:
            raise RuntimeError(f"unknown Int8Linear.mode {self.mode!r} (expected 'tc' or 'sparse')")
        return y.reshape(*orig_shape[:-1], y.shape[-1])

    def extra_repr(self) -> str:
        mode_str = ("sparse_tc (2:4 sparse tcgen05.mma.sp)" if self.mode == "sparse"
                    else "tc_gemm (tcgen05.mma kind::i8)")
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}, mode={mode_str}, epilogue={self.epilogue}")


# ---------------------------------------------------------------------------------------
#  Model surgery (reference: quantize_utils.py:374-498)
# ---------------------------------------------------------------------------------------
def quantize_model_tensorcore(model, min_features=128, verbose=True):
    """Replace ``nn.Linear`` layers with dense ``Int8Linear`` in place.

    Layers with in/out below ``min_features`` are skipped as in the reference; layers that fail
    the kernel's shape rule (K % 64, N % 16) also stay ``nn.Linear`` because there is no
    dequantise fallback to run them (counted under ``kept_fp16``).
    """
    stats = {"total_params": 0, "quantized_params": 0, "skipped_params": 0, "num_replaced": 0}
    _replace_linear_tensorcore(model, min_features, stats)
    if verbose:
        print(_summary(stats, "dense tcgen05 INT8 GEMM", bytes_per_weight=1.0))
    return stats


def _summary(stats, kind, bytes_per_weight):
    """One-paragraph report of a replacement pass (what ``verbose=True`` prints)."""
    q, t = stats["quantized_params"], stats["total_params"]
    kept = stats.get("kept_fp16", 0)
    return (f"  {stats['num_replaced']} nn.Linear -> Int8Linear ({kind}); "
            f"{q / 1e6:.1f}M of {t / 1e6:.1f}M linear weights converted, "
            f"{stats['skipped_params'] / 1e6:.1f}M in layers too small, {kept} layer(s) left as they were; "
            f"weight memory {q * 2 / 1e6:.0f} MB (16-bit) -> {q * bytes_per_weight / 1e6:.0f} MB")


def _replace_linear_tensorcore(module, min_features, stats):
    for name, child in list(module.named_children()):
        if isinstance(child, nn.Linear):
            num_params = child.in_features * child.out_features
            stats["total_params"] += num_params
            if child.in_features < min_features or child.out_features < min_features:
                stats["skipped_params"] += num_params
            elif child.in_features % 64 != 0 or child.out_features % 16 != 0:
                stats["kept_fp16"] = stats.get("kept_fp16", 0) + 1
            else:
                setattr(module, name, Int8Linear.from_linear(child))
                stats["quantized_params"] += num_params
                stats["num_replaced"] += 1
                stats["tc_eligible"] = stats.get("tc_eligible", 0) + 1
        else:
            _replace_linear_tensorcore(child, min_features, stats)


def quantize_model_sparse(model, min_features=128, sparse_min_k=640, verbose=True):
    """Replace ``nn.Linear`` layers with 2:4-sparse ``Int8Linear`` where K >= ``sparse_min_k``;
    other layers stay ``nn.Linear`` (reference: quantize_utils.py:426-498)."""
    sp_available()
    stats = {"total_params": 0, "quantized_params": 0, "skipped_params": 0,
             "num_replaced": 0, "sparse_eligible": 0, "kept_fp16": 0}
    _replace_linear_sparse(model, min_features, sparse_min_k, stats)
    if verbose:
        print(_summary(stats, f"2:4 sparse tcgen05.mma.sp, K >= {sparse_min_k}", bytes_per_weight=0.625))
    return stats


def _replace_linear_sparse(module, min_features, sparse_min_k, stats, choose=None):
    for name, child in list(module.named_children()):
        if isinstance(child, nn.Linear):
            num_params = child.in_features * child.out_features
            stats["total_params"] += num_params
            if child.in_features < min_features or child.out_features < min_features:
                stats["skipped_params"] += num_params
            elif (child.in_features < sparse_min_k or child.in_features % 64 != 0
                  or child.out_features % 16 != 0
                  or (choose is not None and not choose(child.in_features, child.out_features))):
                stats["kept_fp16"] = stats.get("kept_fp16", 0) + 1
            else:
                layer = Int8Linear.from_linear_sparse(child)
                setattr(module, name, layer)
                stats["quantized_params"] += num_params
                stats["num_replaced"] += 1
                if layer._sparse_ok:
                    stats["sparse_eligible"] += 1
        else:
            _replace_linear_sparse(child, min_features, sparse_min_k, stats, choose)


def sparse_pays(in_features: int, out_features: int) -> bool:
    """Whether the 2:4-sparse kernel is the faster one for a layer of this size on B200.
    Measured over the texture UNet's shapes: the sparse GEMM wins where the layer is bound by
    the tensor pipe and shared-memory bandwidth (deep K and many weight rows -- 1280 -> 10240:
    34.7 vs 39.1 us, 5120 -> 1280: 15.8 vs 18.7 us at 3072 tokens) and loses where the output
    write or the per-tile fixed cost dominates (every K <= 640 layer, 1280 -> 320, 1280 -> 1280,
    2560 -> 640).  The reference used one threshold on K (``sparse_min_k=640``, fitted on an
    RTX 4090, quantize_utils.py:426)."""
    return in_features >= 1280 and in_features * out_features >= 5120 * 1280


def quantize_model_mixed(model, min_features=128, sparse_min_k=None, verbose=True):
    """Mixed assignment used by the UNet benchmark: 2:4-sparse layers where that kernel is the
    faster one (``sparse_pays``, or every K >= ``sparse_min_k`` when a threshold is given, as
    in the reference's sparse mode), dense INT8 for every other eligible layer (the
    reference's sparse mode leaves those in fp16, quantize_utils.py:482-489)."""
    sp_available()
    s1 = {"total_params": 0, "quantized_params": 0, "skipped_params": 0,
          "num_replaced": 0, "sparse_eligible": 0, "kept_fp16": 0}
    if sparse_min_k is not None:
        _replace_linear_sparse(model, min_features, sparse_min_k, s1)
    else:
        _replace_linear_sparse(model, min_features, 0, s1, choose=sparse_pays)
    s2 = quantize_model_tensorcore(model, min_features, verbose=False)
    stats = {"sparse_layers": s1["num_replaced"], "dense_layers": s2["num_replaced"],
             "total_params": s1["total_params"],
             "quantized_params": s1["quantized_params"] + s2["quantized_params"],
             "skipped_params": s2["skipped_params"],
             "num_replaced": s1["num_replaced"] + s2["num_replaced"]}
    if verbose:
        print(f"  Quantized {stats['num_replaced']} Linear layers: {stats['sparse_layers']} sparse, "
              f"{stats['dense_layers']} dense")
    return stats


def quantize_model_int8(model, min_features=128, verbose=True):
    """The reference's bitsandbytes mode (quantize_utils.py:505-571) is a memory-only path
    through a third-party library; it is not part of this package."""
    raise RuntimeError("the bitsandbytes mode is not provided; use quantize_model_tensorcore "
                       "or quantize_model_sparse")
