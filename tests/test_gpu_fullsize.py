"""GPU: the benchmark's full-size shapes, checked through size-independent properties (the
CPU oracle would take minutes at these sizes) and on sampled rows against the oracle."""
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"

FULL = list(O.SWEEP_SHAPES)        # all twelve shapes of the sweep


def _case(M, K, N, seed):
    x, w, b = O.make_case(M, K, N, seed)
    wq, ws = O.quantize_weight(w)
    return x, wq, ws.bfloat16(), b


@pytest.mark.parametrize("i,shape", list(enumerate(FULL)))
def test_dense_fullsize_sampled_rows_and_checksum(tc, ik, i, shape):
    M, K, N = shape
    x, wq, ws, b = _case(M, K, N, 100 + i)
    xg, wg = x.to(DEV), wq.to(DEV)
    q, s = ik.fused_quantize_activation(xg)
    acc = tc.int8_gemm_tc(q, wg, None, None, None, out_dtype=torch.int32)
    # (1) sampled rows, bit-exact against the oracle (quantiser + accumulators)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(i))[:257]
    qo, so = O.quantize_activation(x[rows])
    assert torch.equal(q[rows.to(DEV)].cpu(), qo) and torch.equal(s[rows.to(DEV)].cpu(), so)
    assert torch.equal(acc[rows.to(DEV)].cpu(), O.int32_matmul(qo, wq))
    # (2) linearity checksum over ALL rows: sum_m acc[m,:] == (sum_m q[m,:]) @ W^T, exact in int64
    col_sum = acc.to(torch.int64).sum(dim=0).cpu()
    expect = q.to(torch.int64).sum(dim=0).cpu() @ wq.to(torch.int64).t()
    assert torch.equal(col_sum, expect)
    # (3) whole layer (whichever path the library picks) on the sampled rows, inside the 1e-2 gate
    y = tc.int8_linear_tc(xg, wg, ws.to(DEV), b.to(DEV))
    ref = O.epilogue(O.int32_matmul(qo, wq), so, ws, b, torch.bfloat16)
    assert O.rel_l2(y[rows.to(DEV)], ref) < 1e-2
    # (4) the one-launch path, where the kernel takes the shape, gives the same bits
    if K <= 1280:
        assert torch.equal(tc.int8_linear_tc_fused(xg, wg, ws.to(DEV), b.to(DEV)),
                           tc.int8_linear_tc(xg, wg, ws.to(DEV), b.to(DEV), cta_group=1))


@pytest.mark.parametrize("i,shape", [(i, s) for i, s in enumerate(FULL) if s[0] == 49152])
def test_dense_fullsize_every_row_of_the_49152_token_shapes(tc, ik, i, shape):
    """All rows, not a sample: codes, scales and int32 accumulators of the three 49152-token
    layers against the CPU oracle (host int32 matmul of the same int8 tensors)."""
    M, K, N = shape
    x, wq, ws, b = _case(M, K, N, 100 + i)
    q, s = ik.fused_quantize_activation(x.to(DEV))
    qo, so = O.quantize_activation(x)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    acc = tc.int8_gemm_tc(q, wq.to(DEV), None, None, None, out_dtype=torch.int32)
    assert torch.equal(acc.cpu(), O.int32_matmul(qo, wq))
    y = tc.int8_linear_tc(x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV))
    ref = O.epilogue(O.int32_matmul(qo, wq), so, ws, b, torch.bfloat16)
    assert O.rel_l2(y, ref) < 1e-4


@pytest.mark.parametrize("i,shape", list(enumerate(FULL)))
def test_sparse_fullsize_sampled_rows_and_checksum(sp, i, shape):
    M, K, N = shape
    x, wq, ws, b = _case(M, K, N, 200 + i)
    comp, meta = sp.sparse_prune_and_pack(wq.to(DEV))
    co, no = O.prune_compress(wq)
    assert torch.equal(comp.cpu(), co) and torch.equal(meta.cpu(), O.pack_metadata(no, meta.shape[1]))
    wp = O.expand_24(co, no)
    q, s = sp.sparse_quantize_act(x.to(DEV))
    acc = sp.sparse_int8_gemm(q, None, comp, meta, None, None, out_dtype=torch.int32)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(i))[:257]
    assert torch.equal(acc[rows.to(DEV)].cpu(), O.int32_matmul(q[rows.to(DEV)].cpu(), wp))
    col_sum = acc.to(torch.int64).sum(dim=0).cpu()
    assert torch.equal(col_sum, q.to(torch.int64).sum(dim=0).cpu() @ wp.to(torch.int64).t())
    y = sp.sparse_int8_linear(x.to(DEV), comp, meta, ws.to(DEV), b.to(DEV))
    ref = O.epilogue(acc[rows.to(DEV)].cpu(), s[rows.to(DEV)].cpu(), ws, b, torch.bfloat16)
    assert O.rel_l2(y[rows.to(DEV)], ref) < 1e-2
