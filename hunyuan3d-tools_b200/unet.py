"""A self-contained SD2.1-architecture UNet with multiview attention, used as the caller of
the INT8 linear path in the denoise benchmarks.

The reference's model-level tools build ``diffusers.UNet2DConditionModel`` with the
Hunyuan3D-2.1 paint configuration (``tools/test_sparse_unet.py:69-90``,
``tools/test_mixed_vs_all.py:15-24``): channels 320/640/1280/1280, two residual blocks per
level, cross-attention in the first three down levels and the last three up levels, attention
head counts 5/10/20/20 (head_dim 64), 1024-wide conditioning of 77 tokens, linear projections
in the spatial transformers.  ``diffusers`` is not a dependency here, so the same architecture
is written out below from that configuration; weights are random (there are no checkpoints
offline).  On top of it every transformer block gets one multiview self-attention over the
concatenated tokens of all views of a sample, as the texture pipeline's UNet has.

Every ``nn.Linear`` inside is a plain ``nn.Linear`` until
``quantize_utils.quantize_model_{tensorcore,sparse,mixed}`` swaps it, exactly how the
reference treats the upstream UNet (``texture.py:116-131``).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


def timestep_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    """Sinusoidal embedding (flip_sin_to_cos, freq_shift 0 as in SD2.1)."""
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    args = t.float()[:, None] * freqs[None, :]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


class GroupNormNHWC(nn.GroupNorm):
    """``nn.GroupNorm`` (optionally followed by SiLU) that, once ``fused`` is set, runs the
    library's channels-last kernel on channels_last CUDA f16/bf16 inputs: torch's own kernel
    takes NCHW only, so a model whose convolutions run NHWC pays two layout copies around every
    normalisation (14 % of a denoise step, measured).  Parameters and state-dict keys are those
    of ``nn.GroupNorm``; everywhere else (CPU, NCHW, fp32) the torch ops run."""

    def __init__(self, num_groups: int, num_channels: int, eps: float = 1e-5, silu: bool = False):
        super().__init__(num_groups, num_channels, eps=eps)
        self.silu = silu
        self.fused = False
        self._ik = None
        self._ws = None

    def forward(self, x, add=None):
        """``add``: optional (B, C) term added to every pixel before the normalisation (the
        time-embedding projection of a ResNet block); the kernel path adds it on the fly."""
        if (self.fused and x.is_cuda and x.dim() == 4 and x.dtype in (torch.float16, torch.bfloat16)
                and x.is_contiguous(memory_format=torch.channels_last)):
            if self._ik is None:
                from .csrc.build import load_int8_kernels
                self._ik = load_int8_kernels()
            if self._ws is None or self._ws.device != x.device:
                self._ws = torch.empty(1 << 16, dtype=torch.float32, device=x.device)
            return self._ik.groupnorm_nhwc(x, self.num_groups, self.weight, self.bias, self.eps,
                                           silu=self.silu, workspace=self._ws,
                                           add=None if add is None else add.to(x.dtype))
        if add is not None:
            x = x + add[:, :, None, None]
        y = super().forward(x)
        return F.silu(y) if self.silu else y


class ResnetBlock(nn.Module):
    def __init__(self, cin: int, cout: int, temb_dim: int):
        super().__init__()
        self.norm1 = GroupNormNHWC(32, cin, eps=1e-5, silu=True)
        self.conv1 = nn.Conv2d(cin, cout, 3, padding=1)
        self.time_emb_proj = nn.Linear(temb_dim, cout)
        self.norm2 = GroupNormNHWC(32, cout, eps=1e-5, silu=True)
        self.conv2 = nn.Conv2d(cout, cout, 3, padding=1)
        self.conv_shortcut = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x, temb):
        h = self.conv1(self.norm1(x))              # GroupNorm + SiLU
        # h + time embedding feeds norm2 only, so the broadcast add rides in the normalisation
        h = self.conv2(self.norm2(h, add=self.time_emb_proj(F.silu(temb))))
        if self.conv_shortcut is not None:
            x = self.conv_shortcut(x)
        return x + h


class Attention(nn.Module):
    """Multi-head attention with separate q/k/v projections (no bias) and an output
    projection, the layout of diffusers' ``Attention``."""

    def __init__(self, dim: int, heads: int, context_dim: int | None = None):
        super().__init__()
        self.heads = heads
        ctx = context_dim or dim
        self.to_q = nn.Linear(dim, dim, bias=False)
        self.to_k = nn.Linear(ctx, dim, bias=False)
        self.to_v = nn.Linear(ctx, dim, bias=False)
        self.to_out = nn.Linear(dim, dim)
        self.to_qkv = None    # set by fuse_qkv_layers
        self.to_kv = None
        self.is_self = context_dim is None

    def forward(self, x, context=None):
        b, n, c = x.shape
        if self.to_qkv is not None:           # self-attention with the three projections stacked
            q, k, v = self.to_qkv(x).split(c, dim=-1)
            m = n
        else:
            context = x if context is None else context
            m = context.shape[1]
            q = self.to_q(x)
            if self.to_kv is not None:
                k, v = self.to_kv(context).split(c, dim=-1)
            else:
                k, v = self.to_k(context), self.to_v(context)
        q = q.view(b, n, self.heads, c // self.heads).transpose(1, 2)
        k = k.view(b, m, self.heads, c // self.heads).transpose(1, 2)
        v = v.view(b, m, self.heads, c // self.heads).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v)
        return self.to_out(o.transpose(1, 2).reshape(b, n, c))


class GEGLUFeedForward(nn.Module):
    """Linear(C, 8C) -> value * gelu(gate) -> Linear(4C, C).  When the up-projection has been
    converted to an ``Int8Linear`` with the fused GEGLU epilogue it already returns 4C columns."""

    def __init__(self, dim: int):
        super().__init__()
        self.proj = nn.Linear(dim, dim * 8)
        self.out = nn.Linear(dim * 4, dim)

    def forward(self, x):
        h = self.proj(x)
        if h.shape[-1] == self.out.in_features * 2:
            value, gate = h.chunk(2, dim=-1)
            h = value * F.gelu(gate)
        return self.out(h)


class TransformerBlock(nn.Module):
    def __init__(self, dim: int, heads: int, context_dim: int, num_views: int):
        super().__init__()
        self.num_views = num_views
        self.norm1 = nn.LayerNorm(dim)
        self.attn1 = Attention(dim, heads)
        self.norm_mv = nn.LayerNorm(dim)
        self.attn_mv = Attention(dim, heads)          # multiview: all views of a sample at once
        self.norm2 = nn.LayerNorm(dim)
        self.attn2 = Attention(dim, heads, context_dim)
        self.norm3 = nn.LayerNorm(dim)
        self.ff = GEGLUFeedForward(dim)

    def forward(self, x, context):
        x = x + self.attn1(self.norm1(x))
        if self.num_views > 1:
            b, n, c = x.shape
            xv = self.norm_mv(x).view(b // self.num_views, self.num_views * n, c)
            x = x + self.attn_mv(xv).view(b, n, c)
        x = x + self.attn2(self.norm2(x), context)
        return x + self.ff(self.norm3(x))


class SpatialTransformer(nn.Module):
    def __init__(self, dim: int, heads: int, context_dim: int, num_views: int):
        super().__init__()
        self.norm = GroupNormNHWC(32, dim, eps=1e-6)
        self.proj_in = nn.Linear(dim, dim)
        self.block = TransformerBlock(dim, heads, context_dim, num_views)
        self.proj_out = nn.Linear(dim, dim)

    def forward(self, x, context):
        b, c, h, w = x.shape
        y = self.norm(x).permute(0, 2, 3, 1).reshape(b, h * w, c)
        y = self.proj_out(self.block(self.proj_in(y), context))
        return x + y.view(b, h, w, c).permute(0, 3, 1, 2)


class Downsample(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.conv = nn.Conv2d(c, c, 3, stride=2, padding=1)

    def forward(self, x):
        return self.conv(x)


class Upsample(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.conv = nn.Conv2d(c, c, 3, padding=1)

    def forward(self, x):
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


class UNetSD21MV(nn.Module):
    """UNet2DConditionModel of the Hunyuan3D-2.1 paint configuration + multiview attention."""

    def __init__(self, in_channels=4, out_channels=4, block_out_channels=(320, 640, 1280, 1280),
                 layers_per_block=2, attention_heads=(5, 10, 20, 20), cross_attention_dim=1024,
                 num_views=6, attn_levels=(True, True, True, False)):
        super().__init__()
        ch = list(block_out_channels)
        self.num_views = num_views
        temb = ch[0] * 4
        self.time_proj_dim = ch[0]
        self.time_embedding = nn.Sequential(nn.Linear(ch[0], temb), nn.SiLU(), nn.Linear(temb, temb))
        self.conv_in = nn.Conv2d(in_channels, ch[0], 3, padding=1)

        self.down = nn.ModuleList()
        skip_channels = [ch[0]]
        cin = ch[0]
        for lvl, cout in enumerate(ch):
            for _ in range(layers_per_block):
                layer = nn.ModuleDict({"res": ResnetBlock(cin, cout, temb)})
                if attn_levels[lvl]:
                    layer["attn"] = SpatialTransformer(cout, attention_heads[lvl], cross_attention_dim, num_views)
                self.down.append(layer)
                cin = cout
                skip_channels.append(cout)
            if lvl != len(ch) - 1:
                self.down.append(nn.ModuleDict({"down": Downsample(cout)}))
                skip_channels.append(cout)

        self.mid_res1 = ResnetBlock(ch[-1], ch[-1], temb)
        self.mid_attn = SpatialTransformer(ch[-1], attention_heads[-1], cross_attention_dim, num_views)
        self.mid_res2 = ResnetBlock(ch[-1], ch[-1], temb)

        self.up = nn.ModuleList()
        rev = list(reversed(ch))
        rev_attn = list(reversed(attn_levels))
        rev_heads = list(reversed(attention_heads))
        for lvl, cout in enumerate(rev):
            for i in range(layers_per_block + 1):
                skip = skip_channels.pop()
                layer = nn.ModuleDict({"res": ResnetBlock(cin + skip, cout, temb)})
                if rev_attn[lvl]:
                    layer["attn"] = SpatialTransformer(cout, rev_heads[lvl], cross_attention_dim, num_views)
                if i == layers_per_block and lvl != len(rev) - 1:
                    layer["up"] = Upsample(cout)
                self.up.append(layer)
                cin = cout

        self.norm_out = GroupNormNHWC(32, ch[0], eps=1e-5, silu=True)
        self.conv_out = nn.Conv2d(ch[0], out_channels, 3, padding=1)
        # NHWC activations: the convolutions run without layout conversions and the token
        # view (B, H*W, C) the transformer blocks take is free.  Set by use_channels_last().
        self.channels_last = False

    def use_channels_last(self) -> "UNetSD21MV":
        self.to(memory_format=torch.channels_last)
        self.channels_last = True
        return self

    def use_fused_groupnorm(self, on: bool = True) -> "UNetSD21MV":
        """GroupNorm (+ SiLU) through the library's channels-last kernel (CUDA, f16/bf16,
        channels_last activations); elsewhere the torch ops keep running."""
        for m in self.modules():
            if isinstance(m, GroupNormNHWC):
                m.fused = on
        return self

    def forward(self, x, t, context):
        """x: (B*views, 4, H, W); t: (B*views,) or scalar tensor; context: (B*views, 77, 1024)."""
        if t.dim() == 0:
            t = t.expand(x.shape[0])
        temb = self.time_embedding(timestep_embedding(t, self.time_proj_dim).to(x.dtype))
        if self.channels_last:
            x = x.contiguous(memory_format=torch.channels_last)
        h = self.conv_in(x)
        skips = [h]
        for layer in self.down:
            if "down" in layer:
                h = layer["down"](h)
            else:
                h = layer["res"](h, temb)
                if "attn" in layer:
                    h = layer["attn"](h, context)
            skips.append(h)
        h = self.mid_res2(self.mid_attn(self.mid_res1(h, temb), context), temb)
        for layer in self.up:
            h = layer["res"](torch.cat([h, skips.pop()], dim=1), temb)
            if "attn" in layer:
                h = layer["attn"](h, context)
            if "up" in layer:
                h = layer["up"](h)
        return self.conv_out(self.norm_out(h)).contiguous()


def fuse_geglu_layers(model: nn.Module) -> int:
    """Switches every ``Int8Linear`` GEGLU up-projection (dense or 2:4 sparse) to the fused
    ``value * gelu(gate)`` epilogue (rows interleaved offline).  Returns the number fused."""
    from .quantize_utils import Int8Linear
    n = 0
    for m in model.modules():
        if isinstance(m, GEGLUFeedForward) and isinstance(m.proj, Int8Linear) \
                and m.proj.mode in ("tc", "sparse") and m.proj.epilogue == "linear":
            m.proj.interleave_geglu_rows()
            n += 1
    return n


def fuse_layernorm_quant(model: nn.Module) -> int:
    """Replaces the LayerNorms of every transformer block whose consumers are all
    ``Int8Linear`` layers by ``Int8LayerNorm``: norm1 -> stacked q/k/v, norm_mv -> stacked
    multiview q/k/v, norm2 -> cross-attention q, norm3 -> FFN up-projection.  Each of those
    projections then starts from int8 codes emitted by the normalisation kernel instead of
    re-reading and re-quantising its bf16 output.  Run after ``fuse_qkv_layers``.  Returns the
    number of LayerNorms converted."""
    from .quantize_utils import Int8Linear, Int8LayerNorm
    n = 0
    for blk in model.modules():
        if not isinstance(blk, TransformerBlock):
            continue
        pairs = [("norm1", [blk.attn1.to_qkv] if blk.attn1.to_qkv is not None else [blk.attn1.to_q, blk.attn1.to_k, blk.attn1.to_v]),
                 ("norm_mv", [blk.attn_mv.to_qkv] if blk.attn_mv.to_qkv is not None else [blk.attn_mv.to_q, blk.attn_mv.to_k, blk.attn_mv.to_v]),
                 ("norm2", [blk.attn2.to_q]),
                 ("norm3", [blk.ff.proj])]
        for name, consumers in pairs:
            norm = getattr(blk, name)
            if isinstance(norm, nn.LayerNorm) and all(isinstance(c, Int8Linear) for c in consumers):
                setattr(blk, name, Int8LayerNorm(norm))
                n += 1
    return n


def fuse_qkv_layers(model: nn.Module) -> int:
    """Stacks the ``Int8Linear`` projections that read the same activation: q/k/v of every
    self-attention into one layer, k/v of every cross-attention into one.  The activation is
    then quantised once instead of three (two) times and one GEMM replaces three (two); every
    output column keeps its bits.  Returns the number of layers removed."""
    from .quantize_utils import Int8Linear
    removed = 0
    for m in model.modules():
        if not isinstance(m, Attention) or m.to_qkv is not None or m.to_kv is not None:
            continue
        group = [m.to_q, m.to_k, m.to_v] if m.is_self else [m.to_k, m.to_v]
        if not all(isinstance(l, Int8Linear) and l.epilogue == "linear" for l in group):
            continue
        if len({l.mode for l in group}) != 1:
            continue
        fused = Int8Linear.concat(group)
        if m.is_self:
            m.to_qkv, m.to_q, m.to_k, m.to_v = fused, None, None, None
        else:
            m.to_kv, m.to_k, m.to_v = fused, None, None
        removed += len(group) - 1
    return removed


# -----------------------------------------------------------------------------------------
# Denoising loop (deterministic DDIM, classifier-free guidance)
# -----------------------------------------------------------------------------------------
def ddim_alphas(num_train_steps=1000, beta_start=0.00085, beta_end=0.012):
    betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, num_train_steps, dtype=torch.float64) ** 2
    return torch.cumprod(1.0 - betas, dim=0)


def ddim_schedule(steps: int, device):
    """Timesteps and per-step coefficients of the deterministic DDIM update, computed once on
    the host: ``ts`` (steps,) int64 and ``coef`` (steps, 4) fp32 =
    [sqrt(1 - a_t), sqrt(a_t), sqrt(a_prev), sqrt(1 - a_prev)], both on ``device``.  Nothing in
    the step loop has to read a value back from the GPU."""
    acp = ddim_alphas()
    ts = torch.linspace(999, 0, steps + 1).long()[:-1]
    rows = []
    for i, t in enumerate(ts.tolist()):
        a_t = acp[t]
        a_prev = acp[int(ts[i + 1])] if i + 1 < len(ts) else torch.tensor(1.0, dtype=torch.float64)
        rows.append(torch.stack([(1 - a_t).sqrt(), a_t.sqrt(), a_prev.sqrt(), (1 - a_prev).sqrt()]).float())
    return ts.to(device), torch.stack(rows).to(device)


def guided_ddim_update(x: torch.Tensor, eps: torch.Tensor, coef: torch.Tensor, guidance: float):
    """Classifier-free guidance on the [uncond | cond] halves of ``eps`` followed by one DDIM
    update of ``x``; ``coef`` is one row of ``ddim_schedule``.  Pure device arithmetic."""
    eps_u, eps_c = eps.float().chunk(2, dim=0)
    e = eps_u + guidance * (eps_c - eps_u)
    x0 = (x.float() - coef[0] * e) / coef[1]
    return (coef[2] * x0 + coef[3] * e).to(x.dtype)


@torch.no_grad()
def denoise(unet: UNetSD21MV, latents: torch.Tensor, cond: torch.Tensor, uncond: torch.Tensor,
            steps: int = 10, guidance: float = 3.0, step_fn=None) -> torch.Tensor:
    """latents: (views, 4, H, W) of ONE mesh; cond / uncond: (views, 77, 1024).  Each step runs
    the UNet once on the 2 x views batch [uncond | cond] and applies a deterministic DDIM update
    with guidance scale ``guidance`` (3.0 is the texture pipeline's value).  ``step_fn`` lets a
    caller substitute a CUDA-graph replay for the eager UNet call.  The loop issues device work
    only: timesteps and coefficients come from ``ddim_schedule``."""
    ts, coef = ddim_schedule(steps, latents.device)
    context = torch.cat([uncond, cond], dim=0)
    x = latents
    batch = 2 * x.shape[0]
    for i in range(steps):
        t_dev = ts[i].expand(batch)
        inp = torch.cat([x, x], dim=0)
        eps = step_fn(inp, t_dev, context) if step_fn is not None else unet(inp, t_dev, context)
        x = guided_ddim_update(x, eps, coef[i], guidance)
    return x
