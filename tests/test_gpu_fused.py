"""GPU: the dense linear layer as one launch (activations quantised into a resident
shared-memory block) against the two-launch path and the CPU oracle.  Same integer codes and
the same epilogue arithmetic, so every output bit must agree."""
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
    (2000, 1280, 1280),     # one resident block (K > 640), several tiles per block
    (1, 320, 320), (129, 64, 128), (77, 128, 16), (6000, 320, 2560), (257, 96, 48)])
def test_fused_equals_two_launch_path(tc, dtype, M, K, N):
    x, wq, ws, b = _case(M, K, N, dtype, seed=M + K + N)
    xd, wd, sd, bd = x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV)
    y2 = tc.int8_linear_tc(xd, wd, sd, bd, cta_group=1)     # cta_group given: always two launches
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
    y2 = tc.int8_linear_tc(xd, wd, sd, bd, epilogue=code, cta_group=1)
    assert tc.device_status() == 0
    assert torch.equal(y1, y2)
    assert O.rel_l2(y1, O.linear_w8a8(x, wq, ws, b, mode=mode)) < 2e-3


def test_fused_scales_are_the_quantisers(tc, ik):
    """The per-token scales the one-launch kernel reports are the stand-alone quantiser's
    (and the oracle's), ragged last block included."""
    x, wq, ws, b = _case(3000, 1280, 640, torch.bfloat16, seed=9)
    xd, wd, sd, bd = x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV)
    y, s = tc.int8_linear_tc_fused(xd, wd, sd, bd, return_scales=True)
    _, s_ref = ik.fused_quantize_activation(xd)
    assert torch.equal(s, s_ref)
    _, so = O.quantize_activation(x)
    assert torch.equal(s.cpu(), so)
    assert torch.equal(y, tc.int8_linear_tc(xd, wd, sd, bd, cta_group=1))
    assert tc.device_status() == 0


def test_fused_back_to_back_layers(tc):
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
    b = run(lambda *args: tc.int8_linear_tc(*args, cta_group=1))
    assert tc.device_status() == 0
    assert torch.equal(a, b)


@pytest.mark.parametrize("block_n", [32, 64, 128, 160, 192, 256])
def test_fused_tile_widths(tc, block_n):
    x, wq, ws, b = _case(1500, 640, 832, torch.bfloat16, seed=block_n)
    xd, wd, sd, bd = x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV)
    y1 = tc.int8_linear_tc_fused(xd, wd, sd, bd, block_n=block_n)
    y2 = tc.int8_linear_tc(xd, wd, sd, bd, cta_group=1)
    assert tc.device_status() == 0
    assert torch.equal(y1, y2)


def test_fused_many_blocks_per_cta(tc):
    """More token blocks than SMs: every CTA walks several resident blocks (both operand
    buffers and all four scale slots get reused), with a ragged last block."""
    for (M, K, N) in [(148 * 128 * 5 + 77, 320, 320), (148 * 128 * 3 + 1, 1280, 320),
                      (40000, 64, 640), (30000, 1024, 160)]:
        x, wq, ws, b = _case(M, K, N, torch.bfloat16, seed=K)
        xd, wd, sd, bd = x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV)
        y1 = tc.int8_linear_tc_fused(xd, wd, sd, bd)
        y2 = tc.int8_linear_tc(xd, wd, sd, bd, cta_group=1)
        assert tc.device_status() == 0
        assert torch.equal(y1, y2)
        rows = torch.randint(0, M, (300,))
        ref = O.linear_w8a8(x[rows], wq, ws, b)
        assert O.rel_l2(y1[rows.to(DEV)], ref) < 1e-4


def test_default_entry_point_picks_the_path_it_reports(tc):
    """hy3d_linear_w8a8_dense answers with the same bits whichever path it takes, and
    hy3d_linear_path says which one that is."""
    for (M, K, N) in [(148 * 128 + 5, 320, 320), (1000, 320, 320), (20000, 2560, 640)]:
        x, wq, ws, b = _case(M, K, N, torch.bfloat16, seed=3)
        xd, wd, sd, bd = x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV)
        path = tc.int8_linear_path(M, K, N)
        assert path in (0, 1)
        if K > 1280:
            assert path == 0
        y_auto = tc.int8_linear_tc(xd, wd, sd, bd)
        y_two = tc.int8_linear_tc(xd, wd, sd, bd, cta_group=1)
        assert torch.equal(y_auto, y_two)
    assert tc.device_status() == 0


def test_fused_rejects_what_it_cannot_run(tc):
    x, wq, ws, b = _case(300, 2560, 320, torch.bfloat16, seed=1)
    with pytest.raises(RuntimeError):
        tc.int8_linear_tc_fused(x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV))     # K > 1280
    x, wq, ws, b = _case(300, 48, 320, torch.bfloat16, seed=1)
    with pytest.raises(RuntimeError):
        tc.int8_linear_tc_fused(x.to(DEV), wq.to(DEV), ws.to(DEV), b.to(DEV))     # K % 32 != 0
    assert tc.device_status() == 0
