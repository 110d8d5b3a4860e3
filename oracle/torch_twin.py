"""Torch-op twin of one INT8 layer, for model-level parity checks.  TEST INFRASTRUCTURE ONLY.

``OracleInt8Linear`` runs the arithmetic of ``oracle.linear_w8a8`` / ``linear_w8a8_sparse``
(the reference's ``_forward_int_mm`` semantics, quantize_utils.py:293-309, with the CUDA
kernels' epilogue, csrc/int8_sparse_tc.cu:1058-1060) in plain torch ops on whatever device its
input lives on, so a whole UNet whose linears were swapped for it can be evaluated at full
size on a GPU without this repository's kernels.  ``tests/test_oracle.py`` checks it bit for
bit against the CPU oracle functions, which are themselves pinned to the reference's vectors.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import oracle as O


class OracleInt8Linear(nn.Module):
    """Built from a converted layer's buffers: ``weight_int8_nk`` (dense) or
    ``weight_sparse_comp`` + ``weight_sparse_meta`` (2:4 sparse, expanded back to the pruned
    dense matrix), ``weight_scale``, ``bias``, ``epilogue``."""

    def __init__(self, layer):
        super().__init__()
        self.in_features, self.out_features = layer.in_features, layer.out_features
        dev = layer.weight_scale.device
        if layer.mode == "sparse":
            nib = O.unpack_metadata(layer.weight_sparse_meta.cpu(), layer.in_features)
            w = O.expand_24(layer.weight_sparse_comp.cpu(), nib)
        else:
            w = layer.weight_int8_nk.cpu()
        # fp64 holds every int8 product sum exactly (|acc| < 2^53)
        self.register_buffer("w", w.to(dev).double())
        self.register_buffer("scale", layer.weight_scale.float())
        self.bias = None if layer.bias is None else layer.bias.float()
        self.epilogue = layer.epilogue

    def forward(self, x):
        shape = x.shape
        xf = x.reshape(-1, shape[-1]).float()
        amax = xf.abs().amax(dim=1)
        s = torch.clamp(amax, min=1e-8) / torch.full_like(amax, 127.0)
        q = (xf / s[:, None]).round().clamp(-128, 127)
        acc = q.double() @ self.w.t()
        y = acc.float() * (s[:, None] * self.scale[None, :])
        if self.bias is not None:
            y = y + self.bias[None, :]
        if self.epilogue == "gelu":
            y = torch.nn.functional.gelu(y)
        elif self.epilogue == "geglu":
            M, N = y.shape
            y = y.view(M, N // 32, 2, 16)
            y = (y[:, :, 0] * torch.nn.functional.gelu(y[:, :, 1])).reshape(M, N // 2)
        return y.to(x.dtype).reshape(*shape[:-1], y.shape[-1])


def swap_linears(model: nn.Module, layer_type) -> nn.Module:
    """Deep copy of ``model`` with every ``layer_type`` instance replaced by its twin."""
    import copy
    twin = copy.deepcopy(model)

    def swap(mod):
        for name, child in list(mod.named_children()):
            if isinstance(child, layer_type):
                setattr(mod, name, OracleInt8Linear(child))
            elif type(child).__name__ == "Int8LayerNorm":
                # a LayerNorm that emits int8 codes: the twin normalises with the plain torch op
                # and lets the twin layers after it quantise its (rounded) output
                ln = nn.LayerNorm(child.normalized_shape, eps=child.eps)
                ln.weight, ln.bias = child.weight, child.bias
                setattr(mod, name, ln)
            else:
                swap(child)
    swap(twin)
    return twin
