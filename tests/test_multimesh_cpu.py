"""CPU (gloo, world size 2): sharding and collection of independent meshes, including a rank
that fails on one of its meshes."""
import importlib
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_NAME, ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fail_seed, q):
    import sys
    sys.path.insert(0, ROOT)
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    seeds = list(range(7))                      # deliberately not a multiple of the world size
    mine = mm.partition(seeds, rank, world)

    def fake_denoise(seed):                     # stands in for the UNet loop
        if seed == fail_seed:
            raise RuntimeError("injected failure")
        g = torch.Generator().manual_seed(seed)
        return torch.randn(2, 4, 8, 8, generator=g).bfloat16()

    local = mm.run_local(mine, fake_denoise)
    results, missing = mm.gather_results(local, seeds, (2, 4, 8, 8), torch.bfloat16, "cpu", dst=0)
    if rank == 0:
        ok = all(torch.equal(results[s], fake_denoise(s)) for s in results)
        q.put((sorted(results), missing, ok, mine))
    else:
        assert results is None and missing is None
        q.put(("rank1", mine))
    dist.barrier()
    dist.destroy_process_group()


def _run(fail_seed):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, fail_seed, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return out


def test_partition_round_robin(pkg):
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    seeds = list(range(32))
    for world in (1, 2, 4, 8):
        parts = [mm.partition(seeds, r, world) for r in range(world)]
        assert sorted(s for p in parts for s in p) == seeds
        assert all(len(p) == 32 // world for p in parts)
    assert mm.partition(list(range(7)), 1, 2) == [1, 3, 5]


def test_mesh_inputs_are_seeded_and_device_independent(pkg):
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    a = mm.mesh_inputs(3, views=2, size=8, ctx_tokens=5, ctx_dim=16)
    b = mm.mesh_inputs(3, views=2, size=8, ctx_tokens=5, ctx_dim=16)
    c = mm.mesh_inputs(4, views=2, size=8, ctx_tokens=5, ctx_dim=16)
    assert all(torch.equal(x, y) for x, y in zip(a, b)) and not torch.equal(a[0], c[0])
    assert a[0].shape == (2, 4, 8, 8) and a[1].shape == (2, 5, 16) and int(a[2].abs().max()) == 0


def test_gather_two_ranks_all_meshes():
    out = _run(fail_seed=-1)
    rank0 = next(o for o in out if o[0] != "rank1")
    got, missing, ok, mine = rank0
    assert got == list(range(7)) and missing == [] and ok and mine == [0, 2, 4, 6]


def test_gather_reports_meshes_of_a_failing_rank():
    out = _run(fail_seed=3)                      # seed 3 belongs to rank 1
    rank0 = next(o for o in out if o[0] != "rank1")
    got, missing, ok, _ = rank0
    assert got == [0, 1, 2, 4, 5, 6] and missing == [3] and ok


def test_single_process_path(pkg):
    mm = importlib.import_module(PKG_NAME + ".multimesh")
    local = mm.run_local([0, 1], lambda s: torch.full((1,), float(s)))
    res, missing = mm.gather_results(local, [0, 1, 2], (1,), torch.float32)
    assert sorted(res) == [0, 1] and missing == [2]
