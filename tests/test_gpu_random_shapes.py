"""GPU: seeded random problem sizes through the library's own configuration choices (tile
width, CTA pairs, stage depth, tile order, fused quantiser) against the CPU oracle.  Integer
accumulators must be bit-exact for every size, ragged or not."""
import random

import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand_i8(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-128, 128, shape, generator=g, dtype=torch.int8)


def _shapes(seed, n, k_step, n_step, max_m=5000, max_k=5200, max_n=2600):
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        M = rng.choice([rng.randint(1, 300), rng.randint(300, max_m)])
        K = rng.randint(1, max_k // k_step) * k_step
        N = rng.randint(1, max_n // n_step) * n_step
        out.append((M, K, N))
    return out


@pytest.mark.parametrize("M,K,N", _shapes(1234, 24, 16, 16))
def test_dense_random_sizes_bit_exact(tc, M, K, N):
    A, B = _rand_i8((M, K), M * 3 + K), _rand_i8((N, K), N * 5 + K)
    acc = tc.int8_gemm_tc(A.to(DEV), B.to(DEV), None, None, None, out_dtype=torch.int32)
    assert torch.equal(acc.cpu(), O.int32_matmul(A, B))


@pytest.mark.parametrize("M,K,N", _shapes(4321, 16, 64, 16))
def test_sparse_random_sizes_bit_exact(sp, M, K, N):
    X, W = _rand_i8((M, K), M * 7 + K), _rand_i8((N, K), N * 11 + K)
    comp, meta = sp.sparse_prune_and_pack(W.to(DEV))
    acc = sp.sparse_int8_gemm(X.to(DEV), None, comp, meta, None, None, out_dtype=torch.int32)
    co, no = O.prune_compress(W)
    assert torch.equal(comp.cpu(), co)
    assert torch.equal(acc.cpu(), O.int32_matmul(X, O.expand_24(co, no)))


@pytest.mark.parametrize("M,K,N", _shapes(99, 10, 32, 16, max_m=3000, max_k=1280, max_n=1300))
def test_linear_random_sizes_fused_equals_two_launch_and_oracle(tc, M, K, N):
    x, w, b = O.make_case(M, K, N, seed=M + K + N, dtype=torch.bfloat16)
    wq, ws = O.quantize_weight(w)
    ws = ws.bfloat16()
    xd, wd, sd, bd = x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV)
    y2 = tc.int8_linear_tc(xd, wd, sd, bd, cta_group=1)
    y1 = tc.int8_linear_tc_fused(xd, wd, sd, bd)
    assert torch.equal(y1, y2)
    assert O.rel_l2(y2, O.linear_w8a8(x, wq, ws, b)) < 1e-4
    assert tc.device_status() == 0
