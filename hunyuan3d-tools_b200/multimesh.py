"""Multi-mesh texture denoising: independent meshes sharded over GPUs.

The reference textures meshes strictly one after another in a single process
(``texture_batch.py:170-200``); there is no exchange between meshes, so the batch is
data-parallel by construction.  Here one process per GPU (``torchrun``) takes the meshes
``rank, rank + world, ...`` (seeds stand in for meshes: latents and conditioning are generated
from the seed), runs the INT8 UNet denoise loop for each, and rank 0 collects the bf16 latents
with one ``gather``.  No collective sits inside the loop.

The sharding / collection logic is independent of the UNet and is exercised on CPU ranks
(gloo) in the test-suite with a stand-in denoise function; a rank that fails reports which
meshes are missing instead of taking the job down.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Sequence

import torch
import torch.distributed as dist


def partition(items: Sequence[int], rank: int, world: int) -> List[int]:
    """Round-robin assignment: rank r takes items r, r + world, ..."""
    return [items[i] for i in range(rank, len(items), world)]


def mesh_inputs(seed: int, views: int = 6, size: int = 64, ctx_tokens: int = 77, ctx_dim: int = 1024,
                dtype=torch.bfloat16, device="cpu"):
    """Seeded stand-ins for one mesh: initial latents and conditional / unconditional context.
    Generated on the CPU so every device (and the CPU oracle) sees the same bits."""
    g = torch.Generator().manual_seed(seed)
    latents = torch.randn(views, 4, size, size, generator=g).to(dtype)
    cond = torch.randn(views, ctx_tokens, ctx_dim, generator=g).to(dtype)
    uncond = torch.zeros(views, ctx_tokens, ctx_dim).to(dtype)
    return latents.to(device), cond.to(device), uncond.to(device)


def run_local(seeds: Sequence[int], denoise_fn: Callable[[int], torch.Tensor]) -> Dict[int, torch.Tensor]:
    """Runs ``denoise_fn(seed)`` for every local seed; a failing mesh is recorded as missing
    (the reference prints a FAIL line and continues, ``texture_batch.py:196-199``)."""
    done: Dict[int, torch.Tensor] = {}
    for s in seeds:
        try:
            done[s] = denoise_fn(s)
        except Exception as e:  # noqa: BLE001 - reported, the other meshes still run
            print(f"FAIL: mesh {s}: {type(e).__name__}: {e}", flush=True)
    return done


def gather_results(local: Dict[int, torch.Tensor], all_seeds: Sequence[int], example_shape,
                   dtype=torch.bfloat16, device="cpu", dst: int = 0):
    """Collects every rank's finished meshes on ``dst``.

    Returns ``(results, missing)`` on ``dst`` (``results``: seed -> tensor on ``device``;
    ``missing``: seeds nobody delivered) and ``(None, None)`` elsewhere.  Ranks may hold
    different numbers of meshes; each contributes a fixed-size block (its share of
    ``all_seeds``, padded) plus the list of seeds it actually finished.
    """
    if not (dist.is_available() and dist.is_initialized()):
        missing = [s for s in all_seeds if s not in local]
        return dict(local), missing
    rank, world = dist.get_rank(), dist.get_world_size()
    per_rank = (len(all_seeds) + world - 1) // world
    block = torch.zeros((per_rank, *example_shape), dtype=dtype, device=device)
    ids = torch.full((per_rank,), -1, dtype=torch.int64, device=device)
    for i, (s, t) in enumerate(sorted(local.items())):
        block[i].copy_(t)
        ids[i] = s
    blocks = [torch.empty_like(block) for _ in range(world)] if rank == dst else None
    id_lists = [torch.empty_like(ids) for _ in range(world)] if rank == dst else None
    dist.gather(block, blocks, dst=dst)
    dist.gather(ids, id_lists, dst=dst)
    if rank != dst:
        return None, None
    results: Dict[int, torch.Tensor] = {}
    for b, idl in zip(blocks, id_lists):
        for i, s in enumerate(idl.tolist()):
            if s >= 0:
                results[s] = b[i]
    missing = [s for s in all_seeds if s not in results]
    return results, missing


class GraphedStep:
    """One UNet forward captured in a CUDA graph (the reference reaches for
    ``torch.compile(mode="reduce-overhead")`` for the same reason, ``texture.py:141-147``):
    the INT8 layers launch on the current stream and never synchronise, so the whole step
    replays without per-layer host overhead."""

    def __init__(self, unet, batch: int, size: int, ctx_tokens: int, ctx_dim: int, dtype, device):
        self.x = torch.zeros(batch, 4, size, size, dtype=dtype, device=device)
        self.t = torch.zeros(batch, dtype=torch.long, device=device)
        self.ctx = torch.zeros(batch, ctx_tokens, ctx_dim, dtype=dtype, device=device)
        s = torch.cuda.Stream(device=device)
        s.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(s), torch.no_grad():
            for _ in range(2):
                unet(self.x, self.t, self.ctx)
            s.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=s):
                self.out = unet(self.x, self.t, self.ctx)
        torch.cuda.current_stream(device).wait_stream(s)

    def __call__(self, x, t, ctx):
        self.x.copy_(x)
        self.t.copy_(t)
        self.ctx.copy_(ctx)
        self.graph.replay()
        return self.out


class GraphedDenoiser:
    """A whole denoise step -- [x | x] batch, UNet forward, classifier-free guidance, DDIM
    update -- captured once as a CUDA graph.  A mesh is then ten replays with two small
    device-to-device copies in between (timestep and coefficients), no host synchronisation
    and no per-step Python arithmetic on device values."""

    def __init__(self, unet, views: int, size: int, ctx_tokens: int, ctx_dim: int, dtype, device,
                 steps: int = 10, guidance: float = 3.0):
        from .unet import ddim_schedule, guided_ddim_update
        self.steps, self.guidance = steps, guidance
        self.ts, self.coef_all = ddim_schedule(steps, device)
        self.x = torch.zeros(views, 4, size, size, dtype=dtype, device=device)
        self.ctx = torch.zeros(2 * views, ctx_tokens, ctx_dim, dtype=dtype, device=device)
        self.t = torch.zeros(2 * views, dtype=torch.long, device=device)
        self.coef = torch.zeros(4, dtype=torch.float32, device=device)
        self.coef.copy_(self.coef_all[0])

        def one_step():
            eps = unet(torch.cat([self.x, self.x], dim=0), self.t, self.ctx)
            return guided_ddim_update(self.x, eps, self.coef, guidance)

        s = torch.cuda.Stream(device=device)
        s.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(s), torch.no_grad():
            for _ in range(2):
                one_step()
            s.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=s):
                self.x_next = one_step()
        torch.cuda.current_stream(device).wait_stream(s)

    @torch.no_grad()
    def __call__(self, latents, cond, uncond):
        """Enqueues the whole mesh on the current stream and returns the final latents."""
        self.x.copy_(latents, non_blocking=True)
        self.ctx[: uncond.shape[0]].copy_(uncond, non_blocking=True)
        self.ctx[uncond.shape[0]:].copy_(cond, non_blocking=True)
        for i in range(self.steps):
            self.t.copy_(self.ts[i].expand_as(self.t))
            self.coef.copy_(self.coef_all[i])
            self.graph.replay()
            self.x.copy_(self.x_next)
        return self.x.clone()


def build_texture_unet(device, dtype=torch.bfloat16, quant: str = "mixed", seed: int = 0, fuse_geglu=True,
                       fuse_qkv=True, channels_last=True, verbose=False, init_on_device=False,
                       sparse_min_k=None, fuse_ln=True, fused_gn=None, **unet_kwargs):
    """Random-init UNet of the paint configuration with its Linears swapped for INT8 layers.
    ``quant``: "mixed" (2:4 sparse where that kernel is the faster one -- or where
    K >= ``sparse_min_k`` if given -- dense elsewhere), "dense", "sparse" (the
    reference's sparse mode: small-K layers stay bf16) or "none".  ``fuse_qkv`` stacks the
    q/k/v (self-attention) and k/v (cross-attention) projections that share an input.
    ``init_on_device`` draws the random weights on the GPU instead of the CPU.  ``fuse_ln`` lets
    the transformer blocks' LayerNorms emit int8 codes for the projections that follow them.
    ``fused_gn`` runs GroupNorm (+ SiLU) through the library's channels-last kernel (default: on
    for the INT8 modes on a CUDA device with channels_last activations, off for "none", which
    stands for the stock PyTorch model)."""
    from . import quantize_utils as qu
    from .unet import UNetSD21MV, fuse_geglu_layers, fuse_qkv_layers, fuse_layernorm_quant
    torch.manual_seed(seed)
    if init_on_device:
        # Random initialisation by the device's generator: seconds instead of a minute for the
        # 0.9 G parameters, same weights on every GPU of the same type for the same seed.
        with torch.device(device):
            unet = UNetSD21MV(**unet_kwargs)
        unet = unet.to(dtype).eval()
    else:
        unet = UNetSD21MV(**unet_kwargs).to(dtype).to(device).eval()
    if channels_last:
        unet.use_channels_last()
    if fused_gn is None:
        fused_gn = quant != "none"
    if fused_gn and channels_last and torch.device(device).type == "cuda":
        unet.use_fused_groupnorm()
    stats = {}
    if quant == "mixed":
        stats = qu.quantize_model_mixed(unet, sparse_min_k=sparse_min_k, verbose=verbose)
    elif quant == "dense":
        stats = qu.quantize_model_tensorcore(unet, verbose=verbose)
    elif quant == "sparse":
        stats = qu.quantize_model_sparse(unet, verbose=verbose)
    elif quant != "none":
        raise ValueError(f"unknown quant mode {quant!r}")
    if fuse_geglu and quant in ("mixed", "dense", "sparse"):
        stats["geglu_fused"] = fuse_geglu_layers(unet)
    if fuse_qkv and quant != "none":
        stats["qkv_layers_removed"] = fuse_qkv_layers(unet)
    if fuse_ln and quant in ("mixed", "dense"):
        stats["layernorms_emitting_int8"] = fuse_layernorm_quant(unet)
    stats["groupnorms_nhwc_kernel"] = sum(1 for m in unet.modules() if getattr(m, "fused", False) is True)
    return unet, stats


def graphed_denoiser(unet, views: int, size: int, dtype, device, steps: int, guidance: float):
    """The captured step of ``unet`` for this configuration, built on first use and kept on the
    model (two eager forwards plus a capture cost as much as a mesh)."""
    cache = unet.__dict__.setdefault("_graphed_denoisers", {})
    key = (views, size, dtype, str(device), steps, guidance)
    if key not in cache:
        cache[key] = GraphedDenoiser(unet, views, size, 77, 1024, dtype, device, steps, guidance)
    return cache[key]


def denoise_meshes(unet, seeds: Sequence[int], steps: int = 10, guidance: float = 3.0, views: int = 6,
                   size: int = 64, device="cuda", dtype=torch.bfloat16, graphed: bool = True,
                   inputs: Dict[int, tuple] | None = None):
    """Runs the denoise loop for each seed on this rank; returns (seed -> latents, seconds of
    device time measured with CUDA events around the whole loop).  ``inputs`` may hold
    pre-generated (pinned) host tensors per seed, as a data loader would deliver them; missing
    ones are generated on the fly."""
    from .unet import denoise
    den = graphed_denoiser(unet, views, size, dtype, device, steps, guidance) if graphed else None

    def one(seed):
        if inputs is not None and seed in inputs:
            lat, cond, uncond = (t.to(device, non_blocking=True) for t in inputs[seed])
        else:
            lat, cond, uncond = mesh_inputs(seed, views, size, dtype=dtype, device=device)
        if den is not None:
            return den(lat, cond, uncond)
        return denoise(unet, lat, cond, uncond, steps=steps, guidance=guidance)

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    e0.record()
    out = run_local(seeds, one)
    e1.record()
    torch.cuda.synchronize(device)
    return out, e0.elapsed_time(e1) * 1e-3


def prefetch_mesh_inputs(seeds: Sequence[int], views: int = 6, size: int = 64, dtype=torch.bfloat16):
    """Host-side inputs of the given meshes in pinned memory (what a loader thread would have
    ready before the GPU asks for them)."""
    out = {}
    for s in seeds:
        out[s] = tuple(t.pin_memory() if torch.cuda.is_available() else t
                       for t in mesh_inputs(s, views, size, dtype=dtype))
    return out
