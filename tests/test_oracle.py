"""CPU: the oracle against vectors produced by the reference's own CPU code and against the
known-answer cases of its test script."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from conftest import as_half


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_weight_quantisation_matches_reference(golden, tag):
    w = as_half(golden[f"{tag}_weight"])
    q, scale = O.quantize_weight(w)
    assert torch.equal(q, torch.from_numpy(golden[f"{tag}_weight_int8_nk"]))
    assert torch.equal(scale.half(), as_half(golden[f"{tag}_weight_scale"]))


def test_sparse_weight_quantisation_matches_reference(golden):
    w = as_half(golden["s_weight"])
    q, scale = O.quantize_weight(w, sparse_form=True)
    assert torch.equal(q, torch.from_numpy(golden["s_weight_int8"]))
    assert torch.equal(scale.half(), as_half(golden["s_weight_scale"]))
    assert int(q[7].abs().max()) == 0          # the all-zero channel stays zero


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_activation_quantisation_matches_reference(golden, tag):
    x = as_half(golden[f"{tag}_x"])
    q, scale = O.quantize_activation(x)
    assert torch.equal(q, torch.from_numpy(golden[f"{tag}_x_int8"]))


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_int32_accumulators_match_reference(golden, tag):
    q = torch.from_numpy(golden[f"{tag}_x_int8"])
    w = torch.from_numpy(golden[f"{tag}_weight_int8_nk"])
    assert torch.equal(O.int32_matmul(q, w), torch.from_numpy(golden[f"{tag}_acc"]))
    # the fast path and the plain int32 product agree
    assert torch.equal(O.int32_matmul(q, w), q.int() @ w.int().t())


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_linear_output_matches_reference_int_mm_path(golden, tag):
    x = as_half(golden[f"{tag}_x"])
    w8 = torch.from_numpy(golden[f"{tag}_weight_int8_nk"])
    ws = as_half(golden[f"{tag}_weight_scale"])
    b = as_half(golden[f"{tag}_layer_bias"])
    y = O.linear_w8a8(x, w8, ws, b)
    y_ref = as_half(golden[f"{tag}_y_int_mm"])
    # The reference rounds to fp16 before adding the bias, the oracle (like the CUDA
    # kernels) after: at most one fp16 rounding apart.
    assert O.rel_l2(y, y_ref) < 1e-3
    # W8A8 against the reference's fp16-activation dequant path: quantisation error only.
    assert O.rel_l2(y, as_half(golden[f"{tag}_y_dequant"])) < 2e-2


def test_prune_known_answer(golden):
    comp, nib = O.prune_compress(torch.from_numpy(golden["kat_prune_w"]))
    assert torch.equal(comp, torch.from_numpy(golden["kat_prune_comp"]))
    assert torch.equal(nib.reshape(-1), torch.from_numpy(golden["kat_prune_nibbles"]))


def test_prune_tie_rule():
    cases = {
        (5, 5, 5, 5): ((5, 5), 0xE),          # all equal: the later pair survives
        (1, 1, 2, 2): ((2, 2), 0xE),
        (3, -3, 3, 0): ((-3, 3), 0x9),
        (2, 1, 1, 2): ((2, 2), 0xC),
        (-128, 127, 1, 1): ((-128, 127), 0x4),
        (0, 0, 0, 0): ((0, 0), 0xE),
    }
    for g, (kept, nibble) in cases.items():
        comp, nib = O.prune_compress(torch.tensor([list(g)], dtype=torch.int8))
        assert tuple(comp[0].tolist()) == kept and int(nib[0, 0]) == nibble


def test_prune_vectorised_equals_scalar_rule():
    def scalar(v):
        a = [abs(int(t)) for t in v]
        m1, m2 = (1, 0) if a[0] > a[1] else (0, 1)
        for i in (2, 3):
            if a[i] < a[m1]:
                m2, m1 = m1, i
            elif a[i] < a[m2]:
                m2 = i
        keep = [i for i in range(4) if i not in (m1, m2)]
        return [v[keep[0]], v[keep[1]]], keep[0] | (keep[1] << 2)

    g = torch.Generator().manual_seed(5)
    w = torch.randint(-128, 128, (16, 128), dtype=torch.int8, generator=g)
    w[:, :64] = torch.randint(-2, 3, (16, 64), dtype=torch.int8, generator=g)   # many ties
    comp, nib = O.prune_compress(w)
    for r in range(16):
        for k in range(32):
            c, n = scalar(w[r, 4 * k:4 * k + 4].tolist())
            assert c == comp[r, 2 * k:2 * k + 2].tolist() and n == int(nib[r, k])


def test_pack_unpack_expand_roundtrip():
    g = torch.Generator().manual_seed(6)
    w = torch.randint(-128, 128, (48, 320), dtype=torch.int8, generator=g)
    comp, nib = O.prune_compress(w)
    meta = O.pack_metadata(nib, 12)
    assert meta.shape == (48, 12)
    assert torch.equal(O.unpack_metadata(meta, 320), nib)
    assert torch.all(meta[:, 10:] == 0x44444444)
    dense = O.expand_24(comp, nib)
    assert int(((dense.view(48, 80, 4) != 0).sum(-1) > 2).sum()) == 0
    # every surviving value sits where it was, and nothing larger was dropped
    kept = dense != 0
    assert torch.equal(dense[kept], w[kept])
    dropped_max = torch.where(kept, 0, w.int().abs()).view(48, 80, 4).amax(-1)
    kept_min = torch.where(dense.view(48, 80, 4) != 0, dense.view(48, 80, 4).int().abs(), 999).amin(-1)
    assert torch.all(dropped_max <= kept_min)
    # first word = 8 nibbles, least significant first (reference pack_metadata_kernel)
    first = sum(int(nib[0, i]) << (4 * i) for i in range(8))
    assert (int(meta[0, 0]) & 0xFFFFFFFF) == first


def test_sparse_tile_known_answer(golden):
    """The seed-42 random 2:4 tile of the reference's test script: expanding its compressed
    operand with its nibbles and multiplying reproduces the answer it checks against."""
    a_comp = torch.from_numpy(golden["kat_mma_a_comp"])
    nib = torch.from_numpy(golden["kat_mma_nibbles"])
    b = torch.from_numpy(golden["kat_mma_b"])
    c = O.int32_matmul(b, O.expand_24(a_comp, nib)).t()
    assert torch.equal(c, torch.from_numpy(golden["kat_mma_c"]))


def test_epilogue_modes():
    g = torch.Generator().manual_seed(7)
    acc = torch.randint(-100000, 100000, (8, 64), dtype=torch.int32, generator=g)
    a_s = torch.rand(8, generator=g) * 1e-2
    w_s = (torch.rand(64, generator=g) * 1e-3).half()
    b = torch.randn(64, generator=g).half()
    y = O.epilogue(acc, a_s, w_s, b, torch.float16)
    ref = acc.double() * a_s.double()[:, None] * w_s.double()[None, :] + b.double()[None, :]
    assert O.rel_l2(y, ref) < 1e-3
    yg = O.epilogue(acc, a_s, w_s, b, torch.float16, "geglu")
    assert yg.shape == (8, 32)
    lin = O.epilogue(acc, a_s, w_s, b, torch.float32).view(8, 2, 2, 16)
    assert O.rel_l2(yg, (lin[:, :, 0] * torch.nn.functional.gelu(lin[:, :, 1])).reshape(8, 32)) < 1e-3
    perm = O.geglu_interleave_rows(64)
    assert perm[:32].tolist() == list(range(16)) + list(range(32, 48))


def test_zero_row_and_guard():
    x = torch.zeros(2, 16, dtype=torch.float16)
    x[1, 3] = 1.0
    q, s = O.quantize_activation(x)
    assert int(q[0].abs().max()) == 0 and float(s[0]) == pytest.approx(1e-8 / 127.0)
    assert int(q[1, 3]) == 127


def test_torch_twin_equals_the_oracle_layer_bit_for_bit():
    """The torch-op twin used for model-level parity (oracle/torch_twin.py) is a second
    spelling of linear_w8a8 / linear_w8a8_sparse; anchor it to them: same bits on a dense, a
    2:4-sparse and a GEGLU layer, 3-D input included."""
    from types import SimpleNamespace
    from oracle.torch_twin import OracleInt8Linear
    M, K, N = 150, 256, 192
    x, w, b = O.make_case(M, K, N, seed=11, dtype=torch.bfloat16)
    wq, ws = O.quantize_weight(w)
    ws16 = ws.bfloat16()
    dense = SimpleNamespace(in_features=K, out_features=N, mode="tc", epilogue="linear",
                            weight_int8_nk=wq, weight_scale=ws16, bias=b,
                            weight_sparse_comp=None, weight_sparse_meta=None)
    assert torch.equal(OracleInt8Linear(dense)(x), O.linear_w8a8(x, wq, ws16, b))
    assert torch.equal(OracleInt8Linear(dense)(x.view(3, 50, K)).reshape(M, N), O.linear_w8a8(x, wq, ws16, b))
    comp, nib = O.prune_compress(wq)
    sparse = SimpleNamespace(in_features=K, out_features=N, mode="sparse", epilogue="linear",
                             weight_int8_nk=None, weight_scale=ws16, bias=None,
                             weight_sparse_comp=comp, weight_sparse_meta=O.pack_metadata(nib, 4 * ((K + 127) // 128)))
    assert torch.equal(OracleInt8Linear(sparse)(x), O.linear_w8a8_sparse(x, comp, nib, ws16, None))
    perm = O.geglu_interleave_rows(N)
    geglu = SimpleNamespace(in_features=K, out_features=N, mode="tc", epilogue="geglu",
                            weight_int8_nk=wq[perm], weight_scale=ws16[perm], bias=b[perm],
                            weight_sparse_comp=None, weight_sparse_meta=None)
    assert torch.equal(OracleInt8Linear(geglu)(x), O.linear_w8a8(x, wq[perm], ws16[perm], b[perm], mode="geglu"))
