"""GPU: the dense linear layer with the activation quantiser fused into the GEMM kernel
(one launch) against the two-launch path and the CPU oracle.  Integer hand-off, so every
output bit must agree."""
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(M, K, N, dtype, seed):
    x, w, b = O.make_case(M, K, N, seed=seed, dtype=dtype)
    wq, ws = O.quantize_weight(w)
    return x, wq, ws.to(dtype), b


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N", [
    (4096, 320, 1280),      # benchmark config 0: 8 lanes per row, 4 rows per warp batch
    (1000, 640, 320),       # ragged last tile, 16 lanes per row
    (333, 1280, 640),       # 32 lanes per row
    (924, 1024, 320),       # cross-attention K/V shape
    (200, 2560, 640),       # rows read twice (more than 8 vectors per lane)
    (130, 5120, 1280),
    (1, 320, 320), (129, 64, 128), (77, 128, 16), (6000, 320, 2560)])
def test_fused_equals_two_launch_path(tc, dtype, M, K, N):
    x, wq, ws, b = _case(M, K, N, dtype, seed=M + K + N)
    xd, wd, sd, bd = x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV)
    y2 = tc.int8_linear_tc(xd, wd, sd, bd)
    y1 = tc.int8_linear_tc_fused(xd, wd, sd, bd)
    assert tc.device_status() == 0
    assert torch.equal(y1, y2)
    ref = O.linear_w8a8(x, wq, ws, b)
    assert O.rel_l2(y1, ref) < 1e-4


@pytest.mark.parametrize("mode,code", [("gelu", 1), ("geglu", 2)])
def test_fused_epilogues(tc, mode, code):
    x, wq, ws, b = _case(777, 640, 1280, torch.bfloat16, seed=5)
    xd, wd, sd, bd = x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV)
    y1 = tc.int8_linear_tc_fused(xd, wd, sd, bd, epilogue=code)
    y2 = tc.int8_linear_tc(xd, wd, sd, bd, epilogue=code)
    assert tc.device_status() == 0
    assert torch.equal(y1, y2)
    assert O.rel_l2(y1, O.linear_w8a8(x, wq, ws, b, mode=mode)) < 2e-3


def test_fused_workspaces_hold_the_quantiser_output_and_counters_return_to_zero(tc, ik):
    """The int8 codes and scales the fused kernel leaves in its workspaces are the stand-alone
    quantiser's, and the hand-off counters are zero again after every launch (so one buffer
    serves every layer on the stream)."""
    import ctypes
    x, wq, ws, b = _case(3000, 1280, 640, torch.bfloat16, seed=9)
    xd, wd, sd, bd = x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV)
    M, K = x.shape
    N = wq.shape[0]
    q = torch.empty(M, K, dtype=torch.int8, device=DEV)
    s = torch.empty(M, dtype=torch.float32, device=DEV)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    nbytes = int(tc._lib.hy3d_fused_sync_bytes(M))
    assert nbytes == 4 * (2 + (M + 127) // 128)
    sync = torch.zeros(nbytes // 4, dtype=torch.int32, device=DEV)
    for _ in range(3):
        rc = tc._lib.hy3d_linear_w8a8_dense_fused(
            xd.data_ptr(), 1, K, q.data_ptr(), s.data_ptr(), sync.data_ptr(), wd.data_ptr(),
            sd.data_ptr(), 1, bd.data_ptr(), 1, out.data_ptr(), 1, M, N, K, 0, 0,
            torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(sync.abs().sum()) == 0
    q_ref, s_ref = ik.fused_quantize_activation(xd)
    assert torch.equal(q, q_ref) and torch.equal(s, s_ref)
    qo, so = O.quantize_activation(x)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    assert tc.device_status() == 0


def test_fused_back_to_back_layers_share_one_counter_buffer(tc):
    """A chain of layers of different shapes on one stream, launched without host
    synchronisation in between."""
    torch.manual_seed(0)
    shapes = [(2048, 320, 640), (2048, 640, 1280), (2048, 1280, 320), (2048, 320, 320)]
    x0 = torch.randn(2048, 320).bfloat16().to(DEV)
    layers = []
    for (_, K, N) in shapes:
        w = (torch.randn(N, K) * 0.05).bfloat16()
        wq, ws = O.quantize_weight(w)
        layers.append((wq.to(DEV), ws.bfloat16().to(DEV)))
    empty = torch.empty(0, dtype=torch.bfloat16, device=DEV)

    def run(fn):
        h = x0
        for wq, ws in layers:
            h = fn(h, wq, ws, empty)
        return h
    a = run(tc.int8_linear_tc_fused)
    b = run(tc.int8_linear_tc)
    assert tc.device_status() == 0
    assert torch.equal(a, b)


def test_fused_unsupported_combinations_take_the_two_launch_path(tc):
    """Mixed activation / output types are served by the two-launch path of the same entry
    point; the fused kernel itself needs 16-byte aligned rows."""
    x, wq, ws, b = _case(300, 320, 320, torch.float16, seed=1)
    xd, wd, sd, bd = x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV)
    M, K = x.shape
    N = wq.shape[0]
    q = torch.empty(M, K, dtype=torch.int8, device=DEV)
    s = torch.empty(M, dtype=torch.float32, device=DEV)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    sync = torch.zeros(16, dtype=torch.int32, device=DEV)
    rc = tc._lib.hy3d_linear_w8a8_dense_fused(
        xd.data_ptr(), 0, K, q.data_ptr(), s.data_ptr(), sync.data_ptr(), wd.data_ptr(),
        sd.data_ptr(), 0, bd.data_ptr(), 0, out.data_ptr(), 1, M, N, K, 0, 0,
        torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    ref = O.linear_w8a8(x, wq, ws, b).float()
    assert O.rel_l2(out.float(), ref) < 5e-3            # bf16 rounding of an fp16-computed reference
    assert tc.device_status() == 0
