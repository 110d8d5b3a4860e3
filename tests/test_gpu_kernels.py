"""GPU parity tests of the CUDA kernels, called through the C ABI (ctypes binding), against
the CPU oracle.  Integer results must be bit-exact; floating-point outputs are compared with
the tolerance written in each test."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from conftest import as_half

pytestmark = pytest.mark.gpu
DEV = "cuda"


# ------------------------------------------------------------------ activation quantiser
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K", [(257, 320), (1000, 640), (333, 1280), (64, 2560), (77, 5120),
                                 (924, 1024), (9, 64), (5, 8), (3, 16384), (1, 320), (4096, 320)])
def test_quantize_rows_bit_exact(ik, dtype, M, K):
    x, _, _ = O.make_case(M, K, 16, seed=M * 7 + K, dtype=dtype)
    if M > 8:
        x[3] = 0                                   # all-zero token
        x[4] = x[4] * 1e-4                         # tiny row: scale far below 1
    q, s = ik.fused_quantize_activation(x.to(DEV))
    qo, so = O.quantize_activation(x)
    assert torch.equal(s.cpu(), so)
    assert torch.equal(q.cpu(), qo)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_quantizer_rounding_is_exact_for_every_16_bit_input(ik, dtype):
    """The kernel refines x * rcp(scale) instead of dividing.  Its inputs are 16-bit, so the
    claim "codes equal rint(x / scale)" is checked by enumeration on the device: every amax
    pattern x every x pattern with |x| <= amax, against IEEE division."""
    pairs, bad = ik.quantizer_enum_check(dtype)
    assert pairs > 1_000_000_000
    assert bad == 0


def test_quantize_rounding_boundaries(ik):
    """Values that sit exactly on, or one ulp beside, a x.5 quotient."""
    K = 256
    x = torch.zeros(64, K, dtype=torch.float16)
    x[:, 0] = 127.0                                # scale exactly 1
    vals = torch.arange(-126, 126, dtype=torch.float32) + 0.5       # 252 exact ties
    x[0, 1:253] = vals.half()
    x[1, 1:253] = (vals + 0.0625).half()                            # just above the tie
    x[3, 1:253] = (vals - 0.0625).half()                            # just below
    x[2, 0] = 63.5                                 # scale 0.5: every multiple of .25 is a tie
    x[2, 1:] = (torch.arange(K - 1) * 0.25 - 30).half()
    q, s = ik.fused_quantize_activation(x.to(DEV))
    qo, so = O.quantize_activation(x)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)


def test_quantize_matches_reference_golden(ik, golden):
    for tag in "abc":
        x = as_half(golden[f"{tag}_x"])
        q, _ = ik.fused_quantize_activation(x.to(DEV))
        assert torch.equal(q.cpu(), torch.from_numpy(golden[f"{tag}_x_int8"]))


def test_quantize_rejects_bad_arguments(ik):
    with pytest.raises(RuntimeError):
        ik.fused_quantize_activation(torch.zeros(4, 12, dtype=torch.float16, device=DEV))   # K % 8
    with pytest.raises(RuntimeError):
        ik.fused_quantize_activation(torch.zeros(4, 16, dtype=torch.float32, device=DEV))
    q, s = ik.fused_quantize_activation(torch.zeros(0, 64, dtype=torch.float16, device=DEV))
    assert q.shape == (0, 64) and s.shape == (0,)


# ------------------------------------------------------------------ prune / compress / pack
@pytest.mark.parametrize("N,K", [(4, 8), (64, 256), (320, 1280), (1280, 320), (128, 64), (16, 36),
                                 (640, 2560)])
def test_prune_compress_bit_exact(sp, N, K):
    g = torch.Generator().manual_seed(N + K)
    w = torch.randint(-128, 128, (N, K), dtype=torch.int8, generator=g)
    w[:, : K // 2] = torch.randint(-3, 4, (N, K // 2), dtype=torch.int8, generator=g)   # ties
    comp, raw = sp.sparse_prune_compress(w.to(DEV))
    co, no = O.prune_compress(w)
    assert torch.equal(comp.cpu(), co)
    assert raw.shape == (N * K // 4,) and raw.dtype == torch.uint8
    assert torch.equal(raw.cpu().view(N, -1), no)
    if K % 32 == 0:
        comp2, meta = sp.sparse_prune_and_pack(w.to(DEV))
        assert meta.dtype == torch.int32 and meta.shape == (N, 4 * ((K + 127) // 128))
        assert torch.equal(comp2.cpu(), co)
        assert torch.equal(meta.cpu(), O.pack_metadata(no, meta.shape[1]))


def test_prune_known_answer_from_reference_tests(sp, golden):
    comp, raw = sp.sparse_prune_compress(torch.from_numpy(golden["kat_prune_w"]).to(DEV))
    assert torch.equal(comp.cpu(), torch.from_numpy(golden["kat_prune_comp"]))
    assert raw.cpu().tolist() == golden["kat_prune_nibbles"].tolist()


# ------------------------------------------------------------------ dense GEMM
def _rand_i8(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-128, 128, shape, dtype=torch.int8, generator=g)


@pytest.mark.parametrize("M,K,N,bn", [
    (128, 32, 16, 0), (128, 64, 64, 0), (128, 128, 128, 0), (128, 256, 256, 0), (128, 320, 160, 0),
    (100, 320, 320, 0), (256, 640, 640, 0), (4096, 320, 1280, 0), (4096, 320, 1280, 128),
    (777, 1024, 320, 0), (3072, 5120, 1280, 0), (1, 64, 16, 0), (3, 1280, 1280, 0), (31, 192, 48, 0),
    (257, 1536, 1536, 0), (924, 1024, 640, 0), (2000, 320, 2560, 208), (500, 64, 272, 0),
    (130, 16, 16, 0), (640, 2560, 640, 80),
])
def test_dense_accumulators_bit_exact(tc, M, K, N, bn):
    A, B = _rand_i8((M, K), M + K), _rand_i8((N, K), N + K + 1)
    acc = tc.int8_gemm_tc(A.to(DEV), B.to(DEV), None, None, None, out_dtype=torch.int32, block_n=bn)
    assert torch.equal(acc.cpu(), O.int32_matmul(A, B))


@pytest.mark.parametrize("M,K,N,bn", [
    (40000, 192, 256, 0),     # one tile column, 313 row tiles (last one ragged), two K blocks
    (38000, 320, 640, 0),     # three columns of 224; ragged last K block
    (37900, 640, 160, 160),   # five K blocks resident
    (40000, 320, 2560, 256),  # ten columns
])
def test_dense_resident_b_tile_bit_exact(tc, M, K, N, bn):
    """Launches that keep one tile column per CTA with at least two tiles each load their B tile
    once and stream only A (single-CTA tiles; K = 192 / 320 / 640 with two, three and five K
    blocks, ragged last row tile, ragged last K block, one and several tile columns)."""
    A, B = _rand_i8((M, K), M + K + 5), _rand_i8((N, K), N + K + 6)
    acc = tc.int8_gemm_tc(A.to(DEV), B.to(DEV), None, None, None, out_dtype=torch.int32,
                          cta_group=1, block_n=bn)
    assert torch.equal(acc.cpu(), O.int32_matmul(A, B))
    g = torch.Generator().manual_seed(M)
    a_s = torch.rand(M, generator=g) * 0.05 + 1e-3
    w_s = (torch.rand(N, generator=g) * 1e-3 + 1e-5).bfloat16()
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16()
    y = tc.int8_gemm_tc(A.to(DEV), B.to(DEV), a_s.to(DEV), w_s.to(DEV), bias.to(DEV),
                        out_dtype=torch.bfloat16, cta_group=1, block_n=bn)
    ref = O.epilogue(O.int32_matmul(A, B), a_s, w_s, bias, torch.bfloat16, "linear")
    assert O.rel_l2(y, ref) < 2e-3          # same accumulators and formula; fma contraction only
    # and the resident-B launch equals the streaming one bit for bit (pairs stream both operands)
    if K >= 64 and N % 32 == 0:
        y2 = tc.int8_gemm_tc(A.to(DEV), B.to(DEV), a_s.to(DEV), w_s.to(DEV), bias.to(DEV),
                             out_dtype=torch.bfloat16, cta_group=2, block_n=bn)
        assert torch.equal(y, y2)
    assert tc.device_status() == 0


@pytest.mark.parametrize("M,K,N,bn", [
    (2600, 2064, 512, 0),     # K = 8 deep stages + a 16-element tail; ragged last row tile
    (300, 1024, 256, 256),    # exactly four deep stages, second CTA's rows half empty
    (1000, 1104, 320, 160),   # tail of 80: three K steps of the first block
    (513, 5120, 1280, 224),   # ragged tile columns (1280 = 5 x 224 + 160)
    (256, 320, 640, 128),     # short K with pairs: single 128-byte blocks per stage
])
def test_dense_cta_pairs_bit_exact(tc, M, K, N, bn):
    """The CTA-pair variant (cta_group = 2: 256-row tiles; deep two-block stages from K = 1024)."""
    A, B = _rand_i8((M, K), M + K + 2), _rand_i8((N, K), N + K + 3)
    acc = tc.int8_gemm_tc(A.to(DEV), B.to(DEV), None, None, None, out_dtype=torch.int32,
                          cta_group=2, block_n=bn)
    assert torch.equal(acc.cpu(), O.int32_matmul(A, B))
    assert tc.device_status() == 0


def test_dense_extreme_values_no_overflow(tc):
    """|acc| reaches 128*128*K: the int32 accumulators must not saturate or wrap."""
    M, K, N = 128, 5120, 64
    A = torch.full((M, K), -128, dtype=torch.int8)
    B = torch.full((N, K), -128, dtype=torch.int8)
    B[1::2] = 127
    acc = tc.int8_gemm_tc(A.to(DEV), B.to(DEV), None, None, None, out_dtype=torch.int32)
    assert torch.equal(acc.cpu(), A.int() @ B.int().t())
    assert int(acc.max()) == 128 * 128 * K


def test_dense_single_tile_known_answer(tc):
    a = torch.ones(128, 32, dtype=torch.int8)
    b = torch.ones(16, 32, dtype=torch.int8)
    d = tc.test_mma(a.to(DEV), b.to(DEV))
    assert d.shape == (128, 16) and bool((d == 32).all())
    a2, b2 = _rand_i8((128, 128), 1), _rand_i8((256, 128), 2)
    assert torch.equal(tc.test_mma(a2.to(DEV), b2.to(DEV)).cpu(), a2.int() @ b2.int().t())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("mode,code", [("linear", 0), ("gelu", 1), ("geglu", 2)])
@pytest.mark.parametrize("M,K,N", [(300, 320, 1280), (1000, 640, 320), (64, 1280, 2560)])
def test_dense_epilogue_matches_oracle(tc, dtype, mode, code, M, K, N):
    A, B = _rand_i8((M, K), 11), _rand_i8((N, K), 12)
    g = torch.Generator().manual_seed(13)
    a_s = torch.rand(M, generator=g) * 0.05 + 1e-3
    w_s = (torch.rand(N, generator=g) * 1e-3 + 1e-5).to(dtype)
    bias = (torch.randn(N, generator=g) * 0.1).to(dtype)
    y = tc.int8_gemm_tc(A.to(DEV), B.to(DEV), a_s.to(DEV), w_s.to(DEV), bias.to(DEV),
                        out_dtype=dtype, epilogue=code)
    ref = O.epilogue(O.int32_matmul(A, B), a_s, w_s, bias, dtype, mode)
    assert y.shape == ref.shape and y.dtype == dtype
    # same int32 accumulators, same formula: only the final rounding (and fma contraction /
    # erf implementation, ~1e-6) can differ -> far inside the 1e-2 gate
    assert O.rel_l2(y, ref) < 2e-3
    y0 = tc.int8_gemm_tc(A.to(DEV), B.to(DEV), a_s.to(DEV), w_s.to(DEV), torch.empty(0, dtype=dtype, device=DEV),
                         out_dtype=dtype, epilogue=code)
    assert O.rel_l2(y0, O.epilogue(O.int32_matmul(A, B), a_s, w_s, None, dtype, mode)) < 2e-3


def test_dense_linear_config0(tc):
    """Config 0 of the benchmark: X bf16 [4096,320], W bf16 [1280,320], bias bf16 [1280]."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4096, 320, generator=g).bfloat16()
    w = (torch.randn(1280, 320, generator=g) * 0.02).bfloat16()
    b = (torch.randn(1280, generator=g) * 0.01).bfloat16()
    wq, ws = O.quantize_weight(w)
    y = tc.int8_linear_tc(x.to(DEV), wq.to(DEV), ws.bfloat16().to(DEV), b.to(DEV))
    ref = O.linear_w8a8(x, wq, ws.bfloat16(), b)
    assert y.shape == (4096, 1280) and y.dtype == torch.bfloat16
    assert O.rel_l2(y, ref) < 1e-2                      # the stated output gate
    assert O.rel_l2(y, ref) < 1e-4                      # what identical accumulators give
    assert O.rel_l2(y, x.float() @ w.float().t() + b.float()) < 2e-2   # vs unquantised math


def test_dense_rejects_bad_arguments(tc):
    A = torch.zeros(128, 40, dtype=torch.int8, device=DEV)     # K % 16 != 0
    B = torch.zeros(16, 40, dtype=torch.int8, device=DEV)
    with pytest.raises(RuntimeError, match="size|alignment"):
        tc.int8_gemm_tc(A, B, None, None, None, out_dtype=torch.int32)
    A = torch.zeros(128, 64, dtype=torch.int8, device=DEV)
    B = torch.zeros(24, 64, dtype=torch.int8, device=DEV)      # N % 16 != 0
    with pytest.raises(RuntimeError):
        tc.int8_gemm_tc(A, B, None, None, None, out_dtype=torch.int32)
    B = torch.zeros(16, 64, dtype=torch.int8, device=DEV)
    with pytest.raises(RuntimeError):                          # scales missing for a float output
        tc.int8_gemm_tc(A, B, None, None, None, out_dtype=torch.float16)
    with pytest.raises(RuntimeError, match="K mismatch"):
        tc.int8_gemm_tc(A, torch.zeros(16, 128, dtype=torch.int8, device=DEV), None, None, None,
                        out_dtype=torch.int32)


def test_dequant_bias_kernel(ik):
    g = torch.Generator().manual_seed(3)
    acc = torch.randint(-200000, 200000, (257, 320), dtype=torch.int32, generator=g)
    a_s = torch.rand(257, generator=g) * 0.01
    w_s = (torch.rand(320, generator=g) * 1e-3).half()
    b = torch.randn(320, generator=g).half()
    y = ik.fused_dequantize_bias(acc.to(DEV), a_s.to(DEV), w_s.to(DEV), b.to(DEV))
    assert O.rel_l2(y, O.epilogue(acc, a_s, w_s, b, torch.float16)) < 1e-3


# ------------------------------------------------------------------ sparse GEMM
def test_sparse_metadata_layout_probe(sp):
    """X = identity makes the GEMM return the expanded weight itself: every (row, group)
    nibble and every compressed value must land where the 2:4 format says."""
    valid = [0x4, 0x8, 0xC, 0x9, 0xD, 0xE]
    for K in (64, 128, 320):
        N, G = 128, K // 4
        comp = ((torch.arange(K // 2) % 100 + 1)[None, :] + (torch.arange(N) % 20)[:, None]).to(torch.int8)
        nib = torch.tensor([[valid[(r * 7 + g * 5) % 6] for g in range(G)] for r in range(N)],
                           dtype=torch.uint8)
        meta = O.pack_metadata(nib, 4 * ((K + 127) // 128))
        out = sp.sparse_int8_gemm(torch.eye(K, dtype=torch.int8).to(DEV), None, comp.to(DEV),
                                  meta.to(DEV), None, None, out_dtype=torch.int32)
        assert torch.equal(out.cpu(), O.expand_24(comp, nib).int().t().contiguous())


def test_sparse_tile_known_answer_from_reference_tests(sp, golden):
    """The seed-42 random 2:4 tile of the reference's mma.sp test, padded to one tcgen05 tile
    (128 rows, K = 64)."""
    a_comp = torch.zeros(128, 32, dtype=torch.int8)
    a_comp[:16, :16] = torch.from_numpy(golden["kat_mma_a_comp"])
    nib = torch.full((128, 16), 0x4, dtype=torch.uint8)
    nib[:16, :8] = torch.from_numpy(golden["kat_mma_nibbles"])
    b = torch.zeros(16, 64, dtype=torch.int8)
    b[:8, :32] = torch.from_numpy(golden["kat_mma_b"])
    d = sp.test_mma_sp(a_comp.to(DEV), b.to(DEV), O.pack_metadata(nib, 4).to(DEV))
    assert d.shape == (128, 16)
    assert torch.equal(d.cpu()[:16, :8], torch.from_numpy(golden["kat_mma_c"]))
    assert int(d.cpu()[16:].abs().max()) == 0
    ones = sp.test_mma_sp(torch.ones(128, 32, dtype=torch.int8, device=DEV),
                          torch.ones(16, 64, dtype=torch.int8, device=DEV),
                          torch.full((128, 4), 0x44444444, dtype=torch.int32, device=DEV))
    assert bool((ones == 32).all())                  # 32 surviving products per output


@pytest.mark.parametrize("M,K,N,bt", [
    (192, 128, 128, 0), (1000, 640, 640, 0), (3072, 1280, 1280, 0), (924, 1024, 320, 0),
    (4096, 320, 320, 0), (12288, 2560, 640, 240), (3, 1280, 1280, 0), (64, 640, 5120, 0),
    (257, 1536, 4608, 0), (500, 64, 16, 0), (2772, 1024, 320, 128), (1, 64, 16, 0),
    (700, 5120, 1280, 224),
    # deep K, M >= 2048: the CTA-pair variant (256 weight rows per tile), full and ragged tiles
    (2304, 1024, 512, 0), (2100, 2560, 640, 0), (3000, 1280, 1296, 192), (2048, 5120, 1280, 64),
])
def test_sparse_accumulators_bit_exact(sp, M, K, N, bt):
    X, W = _rand_i8((M, K), M + K), _rand_i8((N, K), N + K + 5)
    comp, meta = sp.sparse_prune_and_pack(W.to(DEV))
    acc = sp.sparse_int8_gemm(X.to(DEV), None, comp, meta, None, None, out_dtype=torch.int32,
                              force_tile=bt)
    co, no = O.prune_compress(W)
    assert torch.equal(acc.cpu(), O.int32_matmul(X, O.expand_24(co, no)))


@pytest.mark.parametrize("mode,code", [("linear", 0), ("gelu", 1), ("geglu", 2)])
def test_sparse_pair_variant_epilogues(sp, mode, code):
    """Scaled outputs of the CTA-pair variant (chosen for K >= 1024, M >= 2048)."""
    M, K, N = 2500, 1280, 768
    A, B = _rand_i8((M, K), 31), _rand_i8((N, K), 32)
    g = torch.Generator().manual_seed(33)
    a_s = torch.rand(M, generator=g) * 0.05 + 1e-3
    w_s = (torch.rand(N, generator=g) * 1e-3 + 1e-5).bfloat16()
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16()
    comp, meta = sp.sparse_prune_and_pack(B.to(DEV))
    y = sp.sparse_int8_gemm(A.to(DEV), a_s.to(DEV), comp, meta, w_s.to(DEV), bias.to(DEV),
                            out_dtype=torch.bfloat16, epilogue=code)
    co, no = O.prune_compress(B)
    ref = O.epilogue(O.int32_matmul(A, O.expand_24(co, no)), a_s, w_s, bias, torch.bfloat16, mode)
    assert y.shape == ref.shape
    assert O.rel_l2(y, ref) < 2e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("mode,code", [("linear", 0), ("gelu", 1), ("geglu", 2)])
def test_sparse_epilogue_matches_oracle(sp, dtype, mode, code):
    M, K, N = 500, 640, 1280
    X, W = _rand_i8((M, K), 21), _rand_i8((N, K), 22)
    g = torch.Generator().manual_seed(23)
    a_s = torch.rand(M, generator=g) * 0.05 + 1e-3
    w_s = (torch.rand(N, generator=g) * 1e-3 + 1e-5).to(dtype)
    bias = (torch.randn(N, generator=g) * 0.1).to(dtype)
    comp, meta = sp.sparse_prune_and_pack(W.to(DEV))
    y = sp.sparse_int8_gemm(X.to(DEV), a_s.to(DEV), comp, meta, w_s.to(DEV), bias.to(DEV),
                            out_dtype=dtype, epilogue=code)
    co, no = O.prune_compress(W)
    ref = O.epilogue(O.int32_matmul(X, O.expand_24(co, no)), a_s, w_s, bias, dtype, mode)
    assert y.shape == ref.shape
    assert O.rel_l2(y, ref) < 2e-3


def test_sparse_rejects_bad_arguments(sp):
    X = torch.zeros(64, 96, dtype=torch.int8, device=DEV)          # K % 64 != 0
    comp = torch.zeros(16, 48, dtype=torch.int8, device=DEV)
    meta = torch.zeros(16, 4, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):
        sp.sparse_int8_gemm(X, None, comp, meta, None, None, out_dtype=torch.int32)
    X = torch.zeros(64, 128, dtype=torch.int8, device=DEV)
    comp = torch.zeros(16, 64, dtype=torch.int8, device=DEV)
    with pytest.raises(RuntimeError):                               # wrong metadata pitch
        sp.sparse_int8_gemm(X, None, comp, torch.zeros(16, 8, dtype=torch.int32, device=DEV), None,
                            None, out_dtype=torch.int32)


def test_results_are_deterministic(tc, sp):
    A, B = _rand_i8((2048, 640), 31).to(DEV), _rand_i8((640, 640), 32).to(DEV)
    a_s = torch.rand(2048, device=DEV)
    w_s = torch.rand(640, device=DEV).half()
    first = tc.int8_gemm_tc(A, B, a_s, w_s, None)
    comp, meta = sp.sparse_prune_and_pack(B)
    first_sp = sp.sparse_int8_gemm(A, a_s, comp, meta, w_s, None)
    for _ in range(5):
        assert torch.equal(first, tc.int8_gemm_tc(A, B, a_s, w_s, None))
        assert torch.equal(first_sp, sp.sparse_int8_gemm(A, a_s, comp, meta, w_s, None))


def test_output_canaries_untouched(tc, sp):
    """Ragged sizes: nothing may be written outside the (M,N) result."""
    M, K, N = 130, 320, 48
    A, B = _rand_i8((M, K), 41).to(DEV), _rand_i8((N, K), 42).to(DEV)
    lib = tc._lib
    buf = torch.full((M + 2, N), 0x5A5A5A5A, dtype=torch.int32, device=DEV)
    st = lib.hy3d_gemm_w8a8_dense(A.data_ptr(), B.data_ptr(), None, None, 2, None, 0,
                                  buf[1:].data_ptr(), 3, M, N, K, 0, 0, 0,
                                  torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert bool((buf[0] == 0x5A5A5A5A).all()) and bool((buf[M + 1] == 0x5A5A5A5A).all())
    assert torch.equal(buf[1:M + 1].cpu(), O.int32_matmul(A.cpu(), B.cpu()))


def test_bounded_wait_gives_up_and_reports(tc):
    """A device-side wait that can never be satisfied (one thread on a barrier nobody signals,
    wait limit shortened to 2 ms) ends by itself: the kernel returns, the error word holds the
    wait's code, the stream check raises with the timeout status, and the next ordinary GEMM on
    the same context is exact."""
    lib = tc._lib
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.hy3d_set_wait_limit_ns(2_000_000) == 0
    try:
        assert lib.hy3d_wait_selftest(stream) == 0
        assert lib.hy3d_stream_status(stream) == 5            # HY3D_ERR_TIMEOUT
        with pytest.raises(RuntimeError, match="timed out"):
            tc.check_stream()
        assert tc.device_status() == 0                        # cleared by the raise
    finally:
        assert lib.hy3d_set_wait_limit_ns(0) == 0             # back to the default
    assert lib.hy3d_stream_status(stream) == 0
    A = torch.randint(-128, 128, (300, 256), dtype=torch.int8)
    B = torch.randint(-128, 128, (192, 256), dtype=torch.int8)
    acc = tc.int8_gemm_tc(A.to(DEV), B.to(DEV), None, None, None, out_dtype=torch.int32)
    assert torch.equal(acc.cpu(), O.int32_matmul(A, B))
    tc.check_stream()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K", [(4096, 320), (1000, 640), (333, 1280), (77, 1024), (5, 64), (129, 2048), (2500, 96)])
def test_layernorm_quantize_equals_quantising_its_own_output(ik, dtype, M, K):
    """The fused LayerNorm + quantise kernel: (1) its codes and scales are exactly those of the
    stand-alone quantiser (and of the CPU oracle) applied to the normalised activations it
    reports; (2) those activations are the fp32 LayerNorm rounded to the activation type, to
    within a last-place difference of the torch op."""
    g = torch.Generator().manual_seed(M + K)
    x = (torch.randn(M, K, generator=g) * 3 + 0.5).to(dtype)
    gamma = (1 + 0.1 * torch.randn(K, generator=g)).to(dtype)
    beta = (0.1 * torch.randn(K, generator=g)).to(dtype)
    q, s, y = ik.layernorm_quantize(x.to(DEV), gamma.to(DEV), beta.to(DEV), 1e-5, return_normalised=True)
    q2, s2 = ik.fused_quantize_activation(y)
    assert torch.equal(q, q2) and torch.equal(s, s2)
    qo, so = O.quantize_activation(y.cpu())
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    ref = torch.nn.functional.layer_norm(x.float(), (K,), gamma.float(), beta.float(), 1e-5)
    assert O.rel_l2(y, ref) < (3e-3 if dtype == torch.bfloat16 else 4e-4)       # one output rounding
    assert float((y.float().cpu() - ref).abs().max()) <= (0.04 if dtype == torch.bfloat16 else 0.005) * float(ref.abs().max())
    # without the normalised output the codes are the same
    q3, s3 = ik.layernorm_quantize(x.to(DEV), gamma.to(DEV), beta.to(DEV), 1e-5)
    assert torch.equal(q3, q) and torch.equal(s3, s)


def test_layernorm_quantize_without_affine_and_argument_checks(ik):
    x = torch.randn(64, 256).bfloat16().to(DEV)
    q, s, y = ik.layernorm_quantize(x, None, None, 1e-6, return_normalised=True)
    ref = torch.nn.functional.layer_norm(x.float().cpu(), (256,), None, None, 1e-6)
    assert O.rel_l2(y, ref) < 3e-3
    with pytest.raises(RuntimeError):
        ik.layernorm_quantize(torch.randn(8, 4096).bfloat16().to(DEV), None, None, 1e-5)   # K > 2048


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("silu", [False, True])
@pytest.mark.parametrize("shape", [(2, 320, 32, 32), (3, 640, 16, 16), (2, 960, 16, 16), (1, 1280, 8, 8),
                                   (2, 2560, 8, 8), (1, 64, 5, 7), (12, 320, 64, 64),
                                   (300, 64, 4, 4), (700, 64, 3, 5)])   # more samples than one wave of blocks
def test_groupnorm_nhwc_matches_torch_fp32(ik, dtype, silu, shape):
    """The channels-last GroupNorm (+ SiLU) kernel against torch's ops on the same values:
    fp32 group_norm, rounded to the activation type, then (optionally) fp32 SiLU of the rounded
    value, rounded again -- the two-op sequence the kernel replaces.  Floating point: the
    statistics are summed in another order, so outputs may differ in the last place of the
    16-bit type (tolerance: 3e-3 / 4e-4 relative L2 for bf16 / fp16, and no element off by more
    than two units in the last place of the largest output)."""
    B, C, H, W = shape
    g = torch.Generator().manual_seed(C + H)
    x = (torch.randn(B, C, H, W, generator=g) * 2 + 0.7).to(dtype).to(DEV).contiguous(memory_format=torch.channels_last)
    gamma = (1 + 0.2 * torch.randn(C, generator=g)).to(dtype).to(DEV)
    beta = (0.2 * torch.randn(C, generator=g)).to(dtype).to(DEV)
    y = ik.groupnorm_nhwc(x, 32, gamma, beta, 1e-5, silu=silu)
    assert y.shape == x.shape and y.is_contiguous(memory_format=torch.channels_last)
    ref = torch.nn.functional.group_norm(x.float(), 32, gamma.float(), beta.float(), 1e-5).to(dtype)
    if silu:
        ref = torch.nn.functional.silu(ref.float()).to(dtype)
    assert not torch.isnan(y).any()
    assert O.rel_l2(y, ref) < (3e-3 if dtype == torch.bfloat16 else 4e-4)
    ulp = (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10) * float(ref.float().abs().max())
    assert float((y.float() - ref.float()).abs().max()) <= 2 * ulp
    # in place
    x2 = x.clone(memory_format=torch.channels_last)
    ik.groupnorm_nhwc(x2, 32, gamma, beta, 1e-5, silu=silu, out=x2)
    assert torch.equal(x2, y)
    # with a per-(sample, channel) term added first, rounded as a separate add would store it
    add = (torch.randn(B, C, generator=g) * 0.5).to(dtype).to(DEV)
    ya = ik.groupnorm_nhwc(x, 32, gamma, beta, 1e-5, silu=silu, add=add)
    xa = (x + add[:, :, None, None])
    refa = torch.nn.functional.group_norm(xa.float(), 32, gamma.float(), beta.float(), 1e-5).to(dtype)
    if silu:
        refa = torch.nn.functional.silu(refa.float()).to(dtype)
    assert O.rel_l2(ya, refa) < (3e-3 if dtype == torch.bfloat16 else 4e-4)
    ulpa = (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10) * float(refa.float().abs().max())
    assert float((ya.float() - refa.float()).abs().max()) <= 2 * ulpa


def test_groupnorm_nhwc_argument_checks(ik):
    x = torch.randn(2, 64, 4, 4, device=DEV).bfloat16()
    with pytest.raises(RuntimeError):
        ik.groupnorm_nhwc(x, 32, None, None, 1e-5)                       # NCHW memory
    xl = x.contiguous(memory_format=torch.channels_last)
    y = ik.groupnorm_nhwc(xl, 32, None, None, 1e-5)                      # no affine
    ref = torch.nn.functional.group_norm(xl.float(), 32, None, None, 1e-5)
    assert O.rel_l2(y, ref) < 3e-3
    with pytest.raises(RuntimeError):
        ik.groupnorm_nhwc(torch.randn(1, 60, 4, 4, device=DEV).bfloat16().contiguous(memory_format=torch.channels_last),
                          32, None, None, 1e-5)                          # C % 8, C % groups


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N,splits,epi", [
    (257, 6144, 1536, None, 0),     # the image encoder's deep-K layer: the library's own plan
    (257, 6144, 1536, 5, 1),        # GELU, five ranges (48 K blocks: 10 + 10 + 10 + 10 + 8)
    (100, 3152, 272, 3, 0),         # ragged last K block in the last range, ragged columns
    (924, 1024, 320, 4, 0),         # two stages per range
    (130, 4096, 64, 16, 0),         # one narrow tile column, sixteen ranges
])
def test_dense_splitk_equals_single_launch(tc, dtype, M, K, N, splits, epi):
    """Split-K (int32 partials per K range + reduce/epilogue kernel) gives the bits of the
    single-launch GEMM, whose epilogue it restates, and the int32 sums of the oracle."""
    A, B = _rand_i8((M, K), 31).to(DEV), _rand_i8((N, K), 32).to(DEV)
    g = torch.Generator().manual_seed(33)
    a_s = (torch.rand(M, generator=g) * 0.05 + 1e-3).to(DEV)
    w_s = (torch.rand(N, generator=g) * 1e-3 + 1e-5).to(dtype).to(DEV)
    bias = (torch.randn(N, generator=g) * 0.1).to(dtype).to(DEV)
    if splits is None:
        planned, nbytes = tc.dense_splitk_plan(M, N, K, epi)
        assert planned > 1 and nbytes == planned * ((M + 127) // 128 * 128) * N * 4
    one = tc.int8_gemm_tc(A, B, a_s, w_s, bias, out_dtype=dtype, epilogue=epi, splits=1)
    many = tc.int8_gemm_tc(A, B, a_s, w_s, bias, out_dtype=dtype, epilogue=epi, splits=splits)
    assert torch.equal(one, many)
    ref = O.epilogue(O.int32_matmul(A.cpu(), B.cpu()), a_s.cpu(), w_s.cpu(), bias.cpu(), dtype,
                     "gelu" if epi else "linear")
    assert O.rel_l2(many, ref) < 2e-3
    assert tc.device_status() == 0


def test_dense_splitk_plan_leaves_the_unet_shapes_alone(tc):
    for M, K, N in [(49152, 320, 320), (12288, 640, 5120), (3072, 5120, 1280), (924, 1024, 1280)]:
        assert tc.dense_splitk_plan(M, N, K)[0] == 1
    assert tc.dense_splitk_plan(257, 1536, 6144)[0] > 1
