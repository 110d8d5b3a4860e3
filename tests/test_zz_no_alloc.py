"""GPU: the allocation-free dense linear entry point (scratch kept inside the library) against
the regular one.  Collected last on purpose: a failure here must not hide the other tests."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(M, K, N, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype).to(DEV)
    w = torch.randint(-128, 128, (N, K), dtype=torch.int8, generator=g).to(DEV)
    ws = (torch.rand(N, generator=g) * 1e-3 + 1e-5).to(dtype).to(DEV)
    b = (torch.randn(N, generator=g) * 0.1).to(dtype).to(DEV)
    return x, w, ws, b


def test_static_scratch_matches_regular_entry_point_twice(tc):
    """Two calls in a row share the library's scratch array; the second one is smaller, so
    stale bytes of the first stay behind it in the array and must not leak into the result.
    Both entry points run the same kernels on the same data, so the outputs are identical."""
    for M, K, N, seed, dtype in [(4096, 1280, 640, 1, torch.bfloat16), (777, 320, 2560, 2, torch.float16)]:
        x, w, ws, b = _case(M, K, N, seed, dtype)
        expect = tc.int8_linear_tc(x, w, ws, b)
        out = torch.empty_like(expect)
        got = tc.int8_linear_tc_static(x, w, ws, b, out=out)
        torch.cuda.synchronize()
        assert got.data_ptr() == out.data_ptr()
        assert torch.equal(got, expect)
        assert float((got.float() - expect.float()).abs().max()) == 0.0   # tolerance: none needed


def test_static_scratch_call_leaves_device_memory_as_it_found_it(tc):
    """After a first call (which may load the module's code and resolve the scratch address),
    further calls change neither the caching allocator's figure nor the driver's free-memory
    figure: the entry point allocates nothing."""
    x, w, ws, b = _case(2048, 640, 640, 3, torch.bfloat16)
    out = torch.empty(2048, 640, dtype=torch.bfloat16, device=DEV)
    tc.int8_linear_tc_static(x, w, ws, b, out=out)
    torch.cuda.synchronize()
    allocated, reserved = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        tc.int8_linear_tc_static(x, w, ws, b, out=out)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == allocated and torch.cuda.memory_reserved() == reserved
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_static_scratch_rejects_oversize(tc):
    lib = tc._lib
    max_bytes, max_rows = lib.hy3d_static_scratch_max_bytes(), lib.hy3d_static_scratch_max_rows()
    assert max_bytes == 16 << 20 and max_rows == 65536
    K = 1280
    M = max_bytes // K + 1                       # one row too many for the int8 scratch
    x = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, K, dtype=torch.int8, device=DEV)
    ws = torch.ones(64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="capacity"):
        tc.int8_linear_tc_static(x, w, ws, None)
    x2 = torch.zeros(max_rows + 1, 64, dtype=torch.bfloat16, device=DEV)   # too many rows
    w2 = torch.zeros(64, 64, dtype=torch.int8, device=DEV)
    with pytest.raises(RuntimeError, match="capacity"):
        tc.int8_linear_tc_static(x2, w2, ws, None)
    # at the limit it still runs
    x3 = torch.randn(max_bytes // K, K, device=DEV).bfloat16()
    y = tc.int8_linear_tc_static(x3, w, ws, None)
    assert torch.equal(y, tc.int8_linear_tc(x3, w, ws, None))
