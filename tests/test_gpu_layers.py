"""GPU tests of the host-side module (Int8Linear, model surgery), following the reference's
own integration checks (tools/test_sparse_tc.py:613-693, tools/test_sparse_numerics.py,
tools/test_int8_memory.py) plus parity with vectors from the reference's CPU code."""
import pytest
import torch
import torch.nn as nn

from oracle import oracle as O
from conftest import as_half

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _pruned_dense_weight(layer, sp, w_int8):
    """As tools/test_sparse_numerics.py:39-50: expand the kernel's compressed weight."""
    comp, meta_raw = sp.sparse_prune_compress(w_int8)
    N, K = w_int8.shape
    G = K // 4
    vals = comp.view(N, G, 2).float()
    nib = meta_raw.view(N, G).to(torch.int64)
    idx = torch.stack([nib & 3, (nib >> 2) & 3], dim=-1)
    dense = torch.zeros(N, G, 4, device=w_int8.device)
    dense.scatter_(2, idx, vals)
    assert torch.equal(comp, layer.weight_sparse_comp), "compressed weight mismatch"
    return dense.view(N, K) * layer.weight_scale.float()[:, None]


def test_dense_layer_matches_reference_golden(qu, golden):
    """Same fp16 Linear and inputs the reference's CPU path was run on."""
    for tag, (K, N) in {"a": (320, 128), "b": (128, 256), "c": (1024, 64)}.items():
        lin = nn.Linear(K, N).half()
        lin.weight.data = as_half(golden[f"{tag}_weight"])
        lin.bias.data = as_half(golden[f"{tag}_bias"])
        layer = qu.Int8Linear.from_linear(lin).to(DEV)      # quantised where the reference was: on the CPU
        assert torch.equal(layer.weight_int8_nk.cpu(), torch.from_numpy(golden[f"{tag}_weight_int8_nk"]))
        assert torch.equal(layer.weight_scale.cpu(), as_half(golden[f"{tag}_weight_scale"]))
        y = layer(as_half(golden[f"{tag}_x"]).to(DEV))
        y_ref = as_half(golden[f"{tag}_y_int_mm"])
        assert y.dtype == torch.float16 and y.shape == y_ref.shape
        assert O.rel_l2(y, y_ref) < 1e-2           # output gate against the reference's W8A8 path
        assert O.rel_l2(y, y_ref) < 1e-3           # observed: one fp16 rounding apart
        assert O.rel_l2(y, as_half(golden[f"{tag}_y_dequant"])) < 2e-2


@pytest.mark.parametrize("K,N,M", [(1280, 1280, 64), (1280, 1280, 4096), (320, 1280, 4096),
                                   (1280, 320, 64), (640, 5120, 777)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dense_layer_close_to_fp_linear(qu, K, N, M, dtype):
    """tools/test_int8_memory.py:17-31: rel-L2 < 2 % against the unquantised layer."""
    torch.manual_seed(0)
    lin = nn.Linear(K, N).to(DEV).to(dtype)
    layer = qu.Int8Linear.from_linear(lin)
    x = torch.randn(M, K, device=DEV, dtype=dtype)
    y, ref = layer(x), lin(x)
    assert O.rel_l2(y, ref) < 0.02
    assert O.rel_l2(y, O.linear_w8a8(x.cpu(), layer.weight_int8_nk.cpu(), layer.weight_scale.cpu(),
                                     lin.bias.data.cpu())) < 1e-3


def test_layer_handles_3d_input_and_no_bias(qu):
    """tools/test_sparse_tc.py:646-672."""
    torch.manual_seed(1)
    lin = nn.Linear(640, 1280, bias=False).to(DEV).half()
    for make in (qu.Int8Linear.from_linear, qu.Int8Linear.from_linear_sparse):
        layer = make(lin)
        x = torch.randn(2, 77, 640, device=DEV, dtype=torch.float16)
        y = layer(x)
        assert y.shape == (2, 77, 1280) and not torch.isnan(y).any()
        assert torch.equal(y.view(-1, 1280), layer(x.view(-1, 640)))


def test_sparse_layer_buffers_and_stats(qu, sp):
    """tools/test_sparse_tc.py:628-679: buffer shapes of a 640->1280 layer and the stats of
    quantize_model_sparse on a two-layer MLP."""
    torch.manual_seed(2)
    lin = nn.Linear(640, 1280).to(DEV).half()
    layer = qu.Int8Linear.from_linear_sparse(lin)
    assert layer.mode == "sparse"
    assert tuple(layer.weight_sparse_comp.shape) == (1280, 320)
    assert tuple(layer.weight_sparse_meta.shape) == (1280, 20)      # K/32 words per row
    assert layer.weight_sparse_meta.dtype == torch.int32
    assert layer.weight_int8_nk.numel() == 0
    mlp = nn.Sequential(nn.Linear(640, 1280), nn.GELU(), nn.Linear(1280, 640)).to(DEV).half()
    stats = qu.quantize_model_sparse(mlp, verbose=False)
    assert stats["num_replaced"] == 2 and stats["sparse_eligible"] == 2 and stats["kept_fp16"] == 0
    out = mlp(torch.randn(300, 640, device=DEV, dtype=torch.float16))
    assert out.shape == (300, 640) and not torch.isnan(out).any()
    small = nn.Sequential(nn.Linear(320, 640)).to(DEV).half()
    s2 = qu.quantize_model_sparse(small, verbose=False)
    assert s2["kept_fp16"] == 1 and isinstance(small[0], nn.Linear)


@pytest.mark.parametrize("K,N,M", [(640, 640, 4096), (1280, 1280, 9216), (640, 5120, 2048),
                                   (2560, 640, 4096), (5120, 1280, 1024), (1024, 320, 2772),
                                   (1280, 1280, 3), (1536, 1536, 257), (4096, 1536, 257)])
def test_sparse_layer_numerics(qu, sp, K, N, M):
    """tools/test_sparse_numerics.py:53-76: rel-L2 < 2 % against fp32 math on the pruned
    weights (reduced M for the largest shapes), at M and at 64 rows."""
    torch.manual_seed(0)
    lin = nn.Linear(K, N).to(DEV).half()
    layer = qu.Int8Linear.from_linear_sparse(lin)
    w32 = lin.weight.float()
    scale = w32.abs().amax(dim=1).clamp(min=1e-8) / 127.0
    w_int8 = (w32 / scale[:, None]).round().clamp(-128, 127).to(torch.int8).contiguous()
    w_pruned = _pruned_dense_weight(layer, sp, w_int8)
    for m in sorted({M, 64}):
        x = torch.randn(m, K, device=DEV, dtype=torch.half)
        y = layer(x).float()
        ref = x.float() @ w_pruned.t() + lin.bias.float()
        assert float((y - ref).norm() / ref.norm()) < 0.02
    # and bit-level agreement of the packed buffers with the oracle
    co, no = O.prune_compress(w_int8.cpu())
    assert torch.equal(layer.weight_sparse_comp.cpu(), co)
    assert torch.equal(layer.weight_sparse_meta.cpu(), O.pack_metadata(no, layer.weight_sparse_meta.shape[1]))


def test_geglu_fused_layer(qu):
    torch.manual_seed(3)
    lin = nn.Linear(320, 2560).to(DEV).bfloat16()
    x = torch.randn(1000, 320, device=DEV, dtype=torch.bfloat16)
    plain = qu.Int8Linear.from_linear(lin)
    fused = qu.Int8Linear.from_linear(lin).interleave_geglu_rows()
    v, g = plain(x).float().chunk(2, dim=-1)
    y = fused(x)
    assert y.shape == (1000, 1280)
    # the unfused path rounds value and gate to bf16 first
    assert O.rel_l2(y, v * torch.nn.functional.gelu(g)) < 1e-2


@pytest.mark.parametrize("M", [1000, 3072])
def test_geglu_fused_sparse_layer(qu, M):
    """Row interleaving commutes with 2:4 pruning (which acts along K inside a row), so a
    sparse up-projection can be switched to the fused GEGLU epilogue after conversion; M = 3072
    takes the CTA-pair variant of the sparse kernel."""
    torch.manual_seed(5)
    lin = nn.Linear(1280, 2560).to(DEV).bfloat16()
    x = torch.randn(M, 1280, device=DEV, dtype=torch.bfloat16)
    plain = qu.Int8Linear.from_linear_sparse(lin)
    fused = qu.Int8Linear.from_linear_sparse(lin).interleave_geglu_rows()
    assert fused.mode == "sparse" and fused.epilogue == "geglu"
    v, g = plain(x).float().chunk(2, dim=-1)
    y = fused(x)
    assert y.shape == (M, 1280)
    assert O.rel_l2(y, v * torch.nn.functional.gelu(g)) < 1e-2


def test_mixed_model_surgery(qu):
    torch.manual_seed(4)
    model = nn.Sequential(nn.Linear(320, 1280), nn.Linear(1280, 320), nn.Linear(320, 64)).to(DEV).half()
    stats = qu.quantize_model_mixed(model, sparse_min_k=640, verbose=False)
    assert stats["sparse_layers"] == 1 and stats["dense_layers"] == 1
    assert model[0].mode == "tc" and model[1].mode == "sparse" and isinstance(model[2], nn.Linear)
    y = model(torch.randn(500, 320, device=DEV, dtype=torch.float16))
    assert y.shape == (500, 64) and not torch.isnan(y).any()


def test_kernels_run_on_the_current_stream_and_capture(qu):
    """A layer call is capturable in a CUDA graph (everything is launched on the current
    stream and nothing synchronises)."""
    torch.manual_seed(5)
    layer = qu.Int8Linear.from_linear(nn.Linear(640, 640).to(DEV).half())
    x = torch.randn(512, 640, device=DEV, dtype=torch.float16)
    eager = layer(x)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        layer(x)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            y = layer(x)
    torch.cuda.current_stream().wait_stream(s)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, eager)


def test_sparse_state_dict_roundtrip(qu):
    """A pruned + packed layer reloads into a fresh module without re-pruning (the reference
    cannot: its sparse buffers are registered as None)."""
    torch.manual_seed(7)
    lin = nn.Linear(1280, 640).to(DEV).bfloat16()
    a = qu.Int8Linear.from_linear_sparse(lin)
    sd = {k: v.cpu() if torch.is_tensor(v) else v for k, v in a.state_dict().items()}
    b = qu.Int8Linear(1280, 640, bias=True)
    b.load_state_dict(sd)
    b = b.to(DEV)
    assert b.mode == "sparse" and b.weight_int8_nk.numel() == 0
    assert torch.equal(a.weight_sparse_comp, b.weight_sparse_comp)
    assert torch.equal(a.weight_sparse_meta, b.weight_sparse_meta)
    x = torch.randn(300, 1280, device=DEV, dtype=torch.bfloat16)
    assert torch.equal(a(x), b(x))


def test_host_pipeline_matches_direct_calls(qu, pkg):
    """Layers fed from pinned host memory through the three-stream pipeline return the same
    bits as direct calls on device tensors."""
    import importlib
    host_io = importlib.import_module(pkg.__name__ + ".host_io")
    torch.manual_seed(4)
    shapes = [(1000, 320, 640), (513, 640, 320), (2048, 1280, 1280)]
    layers, hx, hy, ref = [], [], [], []
    for M, K, N in shapes:
        lin = torch.nn.Linear(K, N, device=DEV, dtype=torch.bfloat16)
        L = qu.Int8Linear.from_linear(lin)
        x = torch.randn(M, K).bfloat16()
        layers.append(L)
        hx.append(x.pin_memory())
        hy.append(torch.empty(M, N, dtype=torch.bfloat16).pin_memory())
        ref.append(L(x.to(DEV)).cpu())
    pipe = host_io.HostPipeline(DEV)
    for _ in range(2):
        pipe.run(layers, hx, hy)
    pipe.synchronize()
    for a, b in zip(hy, ref):
        assert torch.equal(a, b)
