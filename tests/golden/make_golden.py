"""Generates tests/golden/reference_cpu.npz by RUNNING the reference's own CPU code.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/Hunyuan3D-Tools

It imports the reference's ``quantize_utils.py`` and calls, on CPU tensors,
``Int8Linear.from_linear``, ``Int8Linear._forward_int_mm`` and ``Int8Linear._forward_dequant`` (each + bias, as ``forward``
does for those modes).  ``torch._int_mm`` is wrapped for the
duration so that the int8 activations, the int8 weight view and the int32 accumulators the
reference produced internally are captured too.  ``Int8Linear.from_linear_sparse`` needs the
reference's CUDA extension for the pruning step; its weight-quantisation half is captured by
handing it a stand-in extension object that records the int8 matrix it is given.

The known-answer cases of the reference's ``tools/test_sparse_tc.py`` (prune pattern
[10,20,1,2] -> [10,20] / nibble 0x4 at lines 202-235; all-ones tile -> 16 at 107-127; the
seed-42 random 2:4 tile at 245-320) are regenerated from their recipes and stored with the
expected answers the script itself computes (dense int32 matmul of the pruned matrix).
"""
import os
import sys

import numpy as np
import torch
import torch.nn as nn


def bits(t: torch.Tensor) -> np.ndarray:
    """fp16 / bf16 tensors are stored as their raw 16-bit patterns."""
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy().copy()
    return t.contiguous().numpy().copy()


def main(ref_root: str):
    sys.path.insert(0, ref_root)
    import quantize_utils as ref  # the reference module, unmodified

    out = {}
    captured = {}
    real_int_mm = torch._int_mm

    def spy_int_mm(a, b):
        r = real_int_mm(a, b)
        captured["a"], captured["b"], captured["acc"] = a.clone(), b.clone(), r.clone()
        return r

    for tag, (M, K, N, seed) in {"a": (64, 320, 128, 0), "b": (3, 128, 256, 1),
                                 "c": (40, 1024, 64, 2)}.items():
        torch.manual_seed(seed)
        lin = nn.Linear(K, N).half()
        x = torch.randn(M, K).half()
        if tag == "a":
            x[5] = 0                      # an all-zero token row
            x[7, 11] = 20.0               # an outlier
        layer = ref.Int8Linear.from_linear(lin)
        torch._int_mm = spy_int_mm
        try:
            y_int_mm = layer._forward_int_mm(x, M) + layer.bias
        finally:
            torch._int_mm = real_int_mm
        y_deq = layer._forward_dequant(x) + layer.bias
        out[f"{tag}_weight"] = bits(lin.weight.data)
        out[f"{tag}_bias"] = bits(lin.bias.data)
        out[f"{tag}_x"] = bits(x)
        out[f"{tag}_weight_int8_nk"] = bits(layer.weight_int8_nk)
        out[f"{tag}_weight_scale"] = bits(layer.weight_scale)
        out[f"{tag}_layer_bias"] = bits(layer.bias)
        out[f"{tag}_x_int8"] = bits(captured["a"][:M])
        out[f"{tag}_acc"] = bits(captured["acc"][:M])
        out[f"{tag}_y_int_mm"] = bits(y_int_mm)
        out[f"{tag}_y_dequant"] = bits(y_deq)

    # Sparse conversion: capture the int8 matrix handed to the pruning extension.
    class Recorder:
        def sparse_prune_and_pack(self, w):
            captured["w_sparse"] = w.clone()
            n, k = w.shape
            return (torch.zeros(n, k // 2, dtype=torch.int8), torch.zeros(n, k // 32, dtype=torch.int32))

    ref._SP_MODULE = Recorder()
    torch.manual_seed(3)
    lin = nn.Linear(640, 128).half()
    lin.weight.data[7] = 0                # an all-zero output channel
    sp_layer = ref.Int8Linear.from_linear_sparse(lin)
    out["s_weight"] = bits(lin.weight.data)
    out["s_weight_int8"] = bits(captured["w_sparse"])
    out["s_weight_scale"] = bits(sp_layer.weight_scale)

    # Model surgery statistics on a toy model (CPU, dense mode; verbose off).
    torch.manual_seed(4)
    toy = nn.Sequential(nn.Linear(256, 512), nn.GELU(), nn.Linear(512, 64), nn.Linear(64, 256),
                        nn.Sequential(nn.Linear(256, 256)))
    stats = ref.quantize_model_tensorcore(toy, min_features=128, verbose=False)
    out["toy_stats"] = np.array([stats["total_params"], stats["quantized_params"],
                                 stats["skipped_params"], stats["num_replaced"],
                                 stats.get("tc_eligible", 0)], dtype=np.int64)

    # Known-answer cases of tools/test_sparse_tc.py.
    w = torch.zeros(4, 8, dtype=torch.int8)
    w[:, 0::4], w[:, 1::4], w[:, 2::4], w[:, 3::4] = 10, 20, 1, 2
    out["kat_prune_w"] = bits(w)
    out["kat_prune_comp"] = np.tile(np.array([10, 20], dtype=np.int8), (4, 2))
    out["kat_prune_nibbles"] = np.full((8,), 0x4, dtype=np.uint8)

    torch.manual_seed(42)
    a_dense = torch.randint(-50, 51, (16, 32), dtype=torch.int8)
    a_pruned = a_dense.clone()
    a_comp = torch.zeros(16, 16, dtype=torch.int8)
    nibbles = torch.zeros(16, 8, dtype=torch.uint8)
    for r in range(16):
        for g in range(8):
            vals = a_dense[r, 4 * g:4 * g + 4].abs()
            _, top2 = vals.topk(2)
            k0, k1 = sorted(top2.tolist())
            for i in range(4):
                if i not in (k0, k1):
                    a_pruned[r, 4 * g + i] = 0
            a_comp[r, 2 * g], a_comp[r, 2 * g + 1] = a_dense[r, 4 * g + k0], a_dense[r, 4 * g + k1]
            nibbles[r, g] = k0 | (k1 << 2)
    b_dense = torch.randint(-30, 31, (8, 32), dtype=torch.int8)
    out["kat_mma_a_comp"] = bits(a_comp)
    out["kat_mma_nibbles"] = bits(nibbles)
    out["kat_mma_b"] = bits(b_dense)
    out["kat_mma_c"] = bits(a_pruned.to(torch.int32) @ b_dense.to(torch.int32).t())

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cpu.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of WizardsForgeGames/Hunyuan3D-Tools>")
    main(sys.argv[1])
