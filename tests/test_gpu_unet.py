"""GPU: the SD2.1-architecture UNet with INT8 linears against the same UNet whose linears run
the oracle's W8A8 arithmetic in plain torch ops (same int8 weights, same activation
quantiser, exact integer matmul, same epilogue formula)."""
import importlib

import pytest
import torch
import torch.nn as nn

from oracle import oracle as O
from conftest import PKG_NAME

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _twin(unet, qu):
    """Same UNet with every INT8 layer replaced by its torch-op twin (oracle/torch_twin.py,
    anchored to the pinned CPU oracle by tests/test_oracle.py)."""
    from oracle.torch_twin import swap_linears
    return swap_linears(unet, qu.Int8Linear)


SMALL = dict(block_out_channels=(128, 256), attention_heads=(2, 4), cross_attention_dim=128,
             num_views=2, attn_levels=(True, True), sparse_min_k=512)   # threshold rule: the reduced
# model has no layer large enough for the measured rule, and the sparse kernel must be on the path


def test_reduced_unet_ten_steps_matches_oracle_linears():
    qu = importlib.import_module(PKG_NAME + ".quantize_utils")
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    un = importlib.import_module(PKG_NAME + ".unet")
    unet, stats = mm.build_texture_unet(DEV, torch.bfloat16, "mixed", seed=0, **SMALL)
    assert stats["sparse_layers"] > 0 and stats["dense_layers"] > 0 and stats["geglu_fused"] > 0
    twin = _twin(unet, qu)
    g = torch.Generator().manual_seed(0)
    lat = torch.randn(2, 4, 16, 16, generator=g).bfloat16().to(DEV)
    cond = torch.randn(2, 7, 128, generator=g).bfloat16().to(DEV)
    uncond = torch.zeros_like(cond)
    # one forward: same inputs, layer-by-layer identical accumulators -> bf16 rounding noise only
    x = torch.cat([lat, lat]); ctx = torch.cat([uncond, cond]); t = torch.full((4,), 500, device=DEV)
    with torch.no_grad():
        y, y_ref = unet(x, t, ctx), twin(x, t, ctx)
    assert not torch.isnan(y).any()
    assert O.rel_l2(y, y_ref) < 2e-2
    a = un.denoise(unet, lat, cond, uncond, steps=10, guidance=3.0)
    b = un.denoise(twin, lat, cond, uncond, steps=10, guidance=3.0)
    assert not torch.isnan(a).any()
    assert O.rel_l2(a, b) < 2e-2          # the stated gate on latents after 10 steps


def test_stacked_qkv_projections_keep_every_bit():
    """q/k/v stacked into one layer: one quantise + one GEMM, outputs bit-identical to the
    separate layers for the dense and the 2:4 sparse kernels."""
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    for quant in ("dense", "mixed"):
        a, sa = mm.build_texture_unet(DEV, torch.bfloat16, quant, seed=2, fuse_qkv=False, **SMALL)
        b, sb = mm.build_texture_unet(DEV, torch.bfloat16, quant, seed=2, fuse_qkv=True, **SMALL)
        assert "qkv_layers_removed" not in sa and sb["qkv_layers_removed"] > 0
        g = torch.Generator().manual_seed(3)
        x = torch.randn(4, 4, 16, 16, generator=g).bfloat16().to(DEV)
        ctx = torch.randn(4, 7, 128, generator=g).bfloat16().to(DEV)
        t = torch.full((4,), 300, device=DEV)
        with torch.no_grad():
            assert torch.equal(a(x, t, ctx), b(x, t, ctx))


def test_graphed_step_equals_eager():
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    un = importlib.import_module(PKG_NAME + ".unet")
    unet, _ = mm.build_texture_unet(DEV, torch.bfloat16, "mixed", seed=1, **SMALL)
    lat, cond, uncond = mm.mesh_inputs(5, views=2, size=16, ctx_tokens=7, ctx_dim=128, device=DEV)
    eager = un.denoise(unet, lat, cond, uncond, steps=3)
    step = mm.GraphedStep(unet, 4, 16, 7, 128, torch.bfloat16, DEV)
    graphed = un.denoise(unet, lat, cond, uncond, steps=3, step_fn=step)
    assert torch.equal(eager, graphed)


def test_full_size_unet_step_runs_and_layer_census():
    """Full paint configuration, 2 x 6 views of 64 x 64 latents: layer counts follow the
    reference's table (tools/profile_unet_shapes.py:32-51 plus four multiview projections per
    transformer block); one step gives finite outputs and agrees with the unquantised model."""
    qu = importlib.import_module(PKG_NAME + ".quantize_utils")
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    unet, stats = mm.build_texture_unet(DEV, torch.bfloat16, "none", seed=0)
    from collections import Counter
    census = Counter((m.in_features, m.out_features) for m in unet.modules() if isinstance(m, nn.Linear))
    assert census[(320, 320)] == 60 and census[(640, 640)] == 60 and census[(1280, 1280)] == 85
    assert census[(320, 2560)] == 5 and census[(640, 5120)] == 5 and census[(1280, 10240)] == 6
    assert census[(1024, 320)] == 10 and census[(1024, 640)] == 10 and census[(1024, 1280)] == 12
    lat, cond, uncond = mm.mesh_inputs(0, device=DEV)
    x = torch.cat([lat, lat]); ctx = torch.cat([uncond, cond]); t = torch.full((12,), 500, device=DEV)
    with torch.no_grad():
        ref = unet(x, t, ctx)
    stats = qu.quantize_model_mixed(unet, verbose=False)
    assert stats["num_replaced"] == 280 and stats["sparse_layers"] == 12    # the 1280-level FFN pairs
    with torch.no_grad():
        y = unet(x, t, ctx)
    assert y.shape == (12, 4, 64, 64) and not torch.isnan(y).any()
    # W8A8 (+2:4 pruning of K >= 640 layers of a random-init net) against bf16: same ballpark
    assert O.rel_l2(y, ref) < 0.5


def test_full_size_unet_ten_steps_matches_oracle_linears():
    """The stated gate at the stated size: full paint configuration (320/640/1280/1280, 6
    views, 64 x 64 latents, CFG batch 2), mixed dense / 2:4-sparse assignment with the GEGLU
    and q/k/v fusions, 10 denoise steps; latents within 2e-2 relative L2 of the same UNet
    whose linears run the oracle's W8A8 arithmetic in torch ops (the size the reference's
    model-level tools run, tools/test_sparse_unet.py:69-90)."""
    qu = importlib.import_module(PKG_NAME + ".quantize_utils")
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    un = importlib.import_module(PKG_NAME + ".unet")
    unet, stats = mm.build_texture_unet(DEV, torch.bfloat16, "mixed", seed=0)
    assert stats["sparse_layers"] > 0 and stats["dense_layers"] > 0 and stats["geglu_fused"] == 16
    twin = _twin(unet, qu)
    lat, cond, uncond = mm.mesh_inputs(0, device=DEV)
    a = un.denoise(unet, lat, cond, uncond, steps=10, guidance=3.0)
    b = un.denoise(twin, lat, cond, uncond, steps=10, guidance=3.0)
    assert a.shape == (6, 4, 64, 64) and not torch.isnan(a).any()
    assert O.rel_l2(a, b) < 2e-2


def test_graphed_denoiser_equals_eager_loop():
    """The whole step (batch build, UNet, guidance, DDIM update) captured once and replayed ten
    times gives the eager loop's latents bit for bit, for two meshes in a row."""
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    un = importlib.import_module(PKG_NAME + ".unet")
    unet, _ = mm.build_texture_unet(DEV, torch.bfloat16, "mixed", seed=1, **SMALL)
    den = mm.GraphedDenoiser(unet, 2, 16, 7, 128, torch.bfloat16, DEV, steps=10, guidance=3.0)
    for seed in (5, 6):
        lat, cond, uncond = mm.mesh_inputs(seed, views=2, size=16, ctx_tokens=7, ctx_dim=128, device=DEV)
        eager = un.denoise(unet, lat, cond, uncond, steps=10, guidance=3.0)
        assert torch.equal(den(lat, cond, uncond), eager)


def test_layernorms_that_emit_int8_keep_the_model_output():
    """With the transformer blocks' LayerNorms emitting int8 codes for the projections behind
    them, the UNet output stays within the model-level gate of the model that normalises with
    the torch op, stores and re-quantises.  (The codes are those of the rounded LayerNorm output;
    the normalisation's own last-place rounding can differ from the torch op, which flips a few
    codes and is amplified by the random-init network.)"""
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    qu = importlib.import_module(PKG_NAME + ".quantize_utils")
    a, sa = mm.build_texture_unet(DEV, torch.bfloat16, "mixed", seed=4, fuse_ln=False, **SMALL)
    b, sb = mm.build_texture_unet(DEV, torch.bfloat16, "mixed", seed=4, fuse_ln=True, **SMALL)
    n_blocks = sum(1 for m in b.modules() if type(m).__name__ == "TransformerBlock")
    assert "layernorms_emitting_int8" not in sa and sb["layernorms_emitting_int8"] == 4 * n_blocks
    assert any(isinstance(m, qu.Int8LayerNorm) for m in b.modules())
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4, 4, 16, 16, generator=g).bfloat16().to(DEV)
    ctx = torch.randn(4, 7, 128, generator=g).bfloat16().to(DEV)
    t = torch.full((4,), 300, device=DEV)
    with torch.no_grad():
        ya, yb = a(x, t, ctx), b(x, t, ctx)
    assert not torch.isnan(yb).any()
    err = O.rel_l2(yb, ya)
    assert err < 2e-2, err          # the gate the configuration states for the model's output


def test_nhwc_groupnorm_kernel_keeps_the_model_output():
    """The UNet with its GroupNorms (+ SiLU) on the library's channels-last kernel against the
    same bf16 model on torch's GroupNorm and SiLU ops, both measured against the fp32 model with
    the same weights: the kernel sums its statistics in another order, which moves last-place
    roundings that the random-init network amplifies, so the two bf16 models differ by about as
    much as either differs from fp32.  Gate: the kernel's model is no further from fp32 than
    1.25 x the torch-op model's distance, and the two bf16 models agree within 3e-2."""
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    un = importlib.import_module(PKG_NAME + ".unet")
    small = {k: v for k, v in SMALL.items() if k != "sparse_min_k"}
    a, sa = mm.build_texture_unet(DEV, torch.bfloat16, "none", seed=4, fused_gn=False, **small)
    b, sb = mm.build_texture_unet(DEV, torch.bfloat16, "none", seed=4, fused_gn=True, **small)
    c, _ = mm.build_texture_unet(DEV, torch.float32, "none", seed=4, fused_gn=False, **small)
    n_gn = sum(1 for m in b.modules() if isinstance(m, un.GroupNormNHWC))
    assert sa["groupnorms_nhwc_kernel"] == 0 and sb["groupnorms_nhwc_kernel"] == n_gn > 0
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4, 4, 16, 16, generator=g).to(DEV)
    ctx = torch.randn(4, 7, 128, generator=g).to(DEV)
    t = torch.full((4,), 300, device=DEV)
    with torch.no_grad():
        ya, yb = a(x.bfloat16(), t, ctx.bfloat16()), b(x.bfloat16(), t, ctx.bfloat16())
        yc = c(x.bfloat16().float(), t, ctx.bfloat16().float())
    assert not torch.isnan(yb).any()
    ea, eb, eab = O.rel_l2(ya, yc), O.rel_l2(yb, yc), O.rel_l2(yb, ya)
    assert eb <= 1.25 * ea + 1e-3, (ea, eb)
    assert eab < 3e-2, eab
    # and the INT8 model runs on the kernel too
    m, sm = mm.build_texture_unet(DEV, torch.bfloat16, "mixed", seed=4, **SMALL)
    assert sm["groupnorms_nhwc_kernel"] == n_gn
    with torch.no_grad():
        ym = m(x.bfloat16(), t, ctx.bfloat16())
    assert not torch.isnan(ym).any()
