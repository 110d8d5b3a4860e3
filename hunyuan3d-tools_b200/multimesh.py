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


def build_texture_unet(device, dtype=torch.bfloat16, quant: str = "mixed", seed: int = 0, fuse_geglu=True,
                       fuse_qkv=True, channels_last=True, verbose=False, **unet_kwargs):
    """Random-init UNet of the paint configuration with its Linears swapped for INT8 layers.
    ``quant``: "mixed" (2:4 sparse where K >= 640, dense elsewhere), "dense", "sparse" (the
    reference's sparse mode: small-K layers stay bf16) or "none".  ``fuse_qkv`` stacks the
    q/k/v (self-attention) and k/v (cross-attention) projections that share an input."""
    from . import quantize_utils as qu
    from .unet import UNetSD21MV, fuse_geglu_layers, fuse_qkv_layers
    torch.manual_seed(seed)
    unet = UNetSD21MV(**unet_kwargs).to(dtype).to(device).eval()
    if channels_last:
        unet.use_channels_last()
    stats = {}
    if quant == "mixed":
        stats = qu.quantize_model_mixed(unet, verbose=verbose)
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
    return unet, stats


def denoise_meshes(unet, seeds: Sequence[int], steps: int = 10, guidance: float = 3.0, views: int = 6,
                   size: int = 64, device="cuda", dtype=torch.bfloat16, graphed: bool = True):
    """Runs the denoise loop for each seed on this rank; returns (seed -> latents, seconds)."""
    from .unet import denoise
    step_fn = GraphedStep(unet, 2 * views, size, 77, 1024, dtype, device) if graphed else None

    def one(seed):
        lat, cond, uncond = mesh_inputs(seed, views, size, dtype=dtype, device=device)
        return denoise(unet, lat, cond, uncond, steps=steps, guidance=guidance, step_fn=step_fn)

    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    out = run_local(seeds, one)
    torch.cuda.synchronize(device)
    return out, time.perf_counter() - t0
