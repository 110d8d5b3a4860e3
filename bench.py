#!/usr/bin/env python
"""Benchmark of the W8A8 linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--quick]
                    [--workload dense_sweep|sparse_sweep|unet|multimesh|one_shape|ref_kernels]

One "step" is one pass over the twelve SD2.1-style texture-UNet linear shapes (M = 2 x 6 views x
tokens per level: 49152 / 12288 / 3072 rows, plus the three cross-attention K/V shapes at
M = 12 x 77): for every shape a whole linear layer, bf16 activations in, per-token quantise,
INT8 tensor-core GEMM, rescale + bias, bf16 out.  Inputs are seeded synthetic tensors with the
configuration's shapes and value distributions (N(0,1) activations with 0.1 % outliers at
20 sigma, N(0,0.02) weights).  `value` is dense-equivalent TOPS (2*M*K*N per layer, summed over
the sweep and over ranks, divided by the slowest rank's time).

With N > 1 every rank runs the sweep on its own (differently seeded) activations -- the tokens
of a different mesh -- with replicated weights and no collective on the data path, so per-GPU
work is fixed ("weak" scaling).  The same JSON line also carries, as sub-records, the other
configurations (2:4-sparse sweep, UNet step, multi-mesh batch), the token-split ("strong")
form of the sweep, a bf16 cuBLAS baseline over the same shapes, and the measured denominators
(INT8 tensor rate, HBM read / write / copy rates); `--quick` leaves the sub-records out.

The timed region replays a CUDA graph of one step; the sweep touches > 1 GB per step, so no
operand survives in the 126 MB L2 from one step to the next.  `--workload one_shape` runs one
entry point a few times on one shape and times nothing: it is the command the profiler
captures under `profiles/` were taken with.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PKG = "hunyuan3d-tools_b200"
SWEEP = [
    (49152, 320, 320), (49152, 320, 2560), (49152, 1280, 320),
    (12288, 640, 640), (12288, 640, 5120), (12288, 2560, 640),
    (3072, 1280, 1280), (3072, 1280, 10240), (3072, 5120, 1280),
    (924, 1024, 320), (924, 1024, 640), (924, 1024, 1280),
]
DINO_SHAPES = [(257, 1536, 1536), (257, 1536, 4608), (257, 1536, 6144), (257, 6144, 1536)]
METRIC = "W8A8 dense/2:4 GEMM TOPS at UNet shapes"
# Average DRAM bytes per GEMM launch of the sweep: the sweep's algorithmic bytes / 12 launches
# (62.8 MB dense, 61.9 MB sparse) times the ratio ncu measured between dram read+write bytes and
# algorithmic bytes on the captured launches (0.71, 0.61 and 0.85 dense, 0.70 and 0.81 sparse:
# reads match the algorithmic figure, part of the output is still in L2 when a kernel ends).
TRAFFIC_BYTES_PER_LAUNCH = {"dense": int(62813660 * 0.72), "sparse": int(61868380 * 0.76)}


def sweep_ops(shapes=SWEEP, frac=1.0):
    return sum(2.0 * int(m * frac) * k * n for m, k, n in shapes)


def make_inputs(shape_idx, M, K, N, seed_base, device, rows=None):
    """Config-1 tensors: x ~ N(0,1) with 0.1 % of entries at +-20, w ~ N(0,0.02), b ~ N(0,0.01)."""
    g = torch.Generator(device="cpu").manual_seed(seed_base + shape_idx)
    rows = M if rows is None else rows
    x = torch.randn(rows, K, generator=g)
    mask = torch.rand(rows, K, generator=g) < 0.001
    sign = torch.where(torch.rand(rows, K, generator=g) < 0.5, -1.0, 1.0)
    x = torch.where(mask, 20.0 * sign, x).bfloat16()
    gw = torch.Generator(device="cpu").manual_seed(100 + shape_idx)      # weights: same on every rank
    w = (torch.randn(N, K, generator=gw) * 0.02).bfloat16()
    b = (torch.randn(N, generator=gw) * 0.01).bfloat16()
    return x.to(device), w.to(device), b.to(device)


def env_knobs():
    """Environment variables the library or this script read; printed with every result so a
    number taken under a non-default setting can be told apart."""
    return {k: v for k, v in sorted(os.environ.items()) if k.startswith("HY3D_")}


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except Exception:
        return {}


# ---------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only)."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index):
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _once(self):
        nv = self._nv
        self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
        try:
            self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
        except Exception:
            try:
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
            except Exception:
                r = 0
        for bit, name in self.REASONS.items():
            if r & bit:
                self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                self._once()
            except Exception:
                return
            time.sleep(0.005)

    def start(self):
        if self._nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s), "samples_in_timed_region": len(s),
                "power_w_max": max(self.power) if self.power else None}


# ---------------------------------------------------------------------------------------
# timing helpers
# ---------------------------------------------------------------------------------------
class Ctx:
    """Per-process set-up shared by every workload."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.qu = importlib.import_module(PKG + ".quantize_utils")
        build = importlib.import_module(PKG + ".csrc.build")
        self.tc = build.load_tc_gemm()
        self.sp = build.load_sparse_tc()
        self.lib = self.tc._lib
        self.stream = torch.cuda.Stream(device=self.dev)

    def max_over_ranks(self, v: float) -> float:
        if self.dist is None:
            return v
        t = torch.tensor([v], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


def capture(ctx: Ctx, fn):
    """fn(stream_handle) launches a sequence of kernels; returns a CUDA graph of it."""
    with torch.cuda.stream(ctx.stream):
        fn(ctx.stream.cuda_stream)                       # first call outside capture (lazy set-up)
        ctx.stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=ctx.stream):
            fn(ctx.stream.cuda_stream)
    return g


def timed_repeats(ctx: Ctx, replay, steps, warmup, repeats=5, sampler=None):
    """`repeats` timed regions of `steps` replays each (CUDA events on the launching stream,
    barrier + synchronize on both sides, max over ranks); returns ms per step of every repeat."""
    out = []
    with torch.cuda.stream(ctx.stream):
        for _ in range(warmup):
            replay()
        ctx.stream.synchronize()
        if sampler:
            sampler.start()
        for _ in range(repeats):
            ctx.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(ctx.stream)
            for _ in range(steps):
                replay()
            e1.record(ctx.stream)
            torch.cuda.synchronize()
            ctx.barrier()
            out.append(ctx.max_over_ranks(e0.elapsed_time(e1)) / steps)
        if sampler:
            sampler.stop()
    return out


def spread(xs, digits=4):
    return {"median": round(statistics.median(xs), digits), "min": round(min(xs), digits),
            "max": round(max(xs), digits), "repeats": len(xs)}


# ---------------------------------------------------------------------------------------
# the sweep
# ---------------------------------------------------------------------------------------
class Sweep:
    """The twelve layers with pre-allocated workspaces and outputs, so that a step is pure
    kernel launches through the C ABI (the entry points Int8Linear.forward uses).
    `row_range` = (lo, hi) fractions of every shape's M for the token-split form."""

    def __init__(self, ctx: Ctx, sparse: bool, seed_base: int, row_range=(0.0, 1.0), shapes=SWEEP):
        self.ctx, self.sparse = ctx, sparse
        dev, qu = ctx.dev, ctx.qu
        self.layers, self.xs, self.raw = [], [], []
        for i, (M, K, N) in enumerate(shapes):
            lo, hi = int(M * row_range[0]), int(M * row_range[1])
            x, w, b = make_inputs(i, M, K, N, seed_base, dev)
            x = x[lo:hi].contiguous()
            lin = torch.nn.Linear(K, N, device=dev, dtype=torch.bfloat16)
            lin.weight.data.copy_(w)
            lin.bias.data.copy_(b)
            self.layers.append((qu.Int8Linear.from_linear_sparse if sparse else qu.Int8Linear.from_linear)(lin))
            self.xs.append(x)
            self.raw.append((hi - lo, K, N))
        self.ops = sum(2.0 * m * k * n for m, k, n in self.raw)
        self.qs = [torch.empty((M, K), dtype=torch.int8, device=dev) for M, K, N in self.raw]
        self.ss = [torch.empty((M,), dtype=torch.float32, device=dev) for M, K, N in self.raw]
        self.outs = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for M, K, N in self.raw]

    def linear(self, i, stream):
        M, K, N = self.raw[i]
        L, lib = self.layers[i], self.ctx.lib
        if self.sparse:
            st = lib.hy3d_linear_w8a8_sparse24(
                self.xs[i].data_ptr(), 1, K, self.qs[i].data_ptr(), self.ss[i].data_ptr(),
                L.weight_sparse_comp.data_ptr(), L.weight_sparse_meta.data_ptr(),
                L.weight_sparse_meta.shape[1], L.weight_scale.data_ptr(), 1, L.bias.data_ptr(), 1,
                self.outs[i].data_ptr(), 1, M, N, K, 0, 0, stream)
        else:
            st = lib.hy3d_linear_w8a8_dense(
                self.xs[i].data_ptr(), 1, K, self.qs[i].data_ptr(), self.ss[i].data_ptr(),
                L.weight_int8_nk.data_ptr(), L.weight_scale.data_ptr(), 1, L.bias.data_ptr(), 1,
                self.outs[i].data_ptr(), 1, M, N, K, 0, 0, 0, stream)
        if st != 0:
            raise RuntimeError(f"linear launch failed with status {st}")

    def gemm_only(self, i, stream):
        M, K, N = self.raw[i]
        L, lib = self.layers[i], self.ctx.lib
        if self.sparse:
            st = lib.hy3d_gemm_w8a8_sparse24(
                self.qs[i].data_ptr(), self.ss[i].data_ptr(), L.weight_sparse_comp.data_ptr(),
                L.weight_sparse_meta.data_ptr(), L.weight_sparse_meta.shape[1],
                L.weight_scale.data_ptr(), 1, L.bias.data_ptr(), 1, self.outs[i].data_ptr(), 1, M, N, K,
                0, 0, stream)
        else:
            st = lib.hy3d_gemm_w8a8_dense(
                self.qs[i].data_ptr(), L.weight_int8_nk.data_ptr(), self.ss[i].data_ptr(),
                L.weight_scale.data_ptr(), 1, L.bias.data_ptr(), 1, self.outs[i].data_ptr(), 1, M, N, K,
                0, 0, 0, stream)
        if st != 0:
            raise RuntimeError(f"gemm launch failed with status {st}")

    def quant_only(self, i, stream):
        M, K, N = self.raw[i]
        st = self.ctx.lib.hy3d_quantize_rows(self.xs[i].data_ptr(), 1, M, K, K, self.qs[i].data_ptr(),
                                             self.ss[i].data_ptr(), stream)
        if st != 0:
            raise RuntimeError(f"quantise launch failed with status {st}")

    def graphs(self):
        n = len(self.raw)
        g_step = capture(self.ctx, lambda s: [self.linear(i, s) for i in range(n)])
        g_gemm = capture(self.ctx, lambda s: [self.gemm_only(i, s) for i in range(n)])
        return g_step, g_gemm


def measured_denominators(ctx: Ctx):
    """INT8 tensor rate (resident-operand tcgen05.mma issue loop on every SM) and HBM stream
    rates, measured with this library's probes on this GPU, right now."""
    lib, dev = ctx.lib, ctx.dev
    out = {}
    cur = torch.cuda.current_stream().cuda_stream
    import ctypes
    for name, n, sparse in (("int8_dense_tops", 256, 0), ("int8_sparse24_tops", 240, 1)):
        ops = ctypes.c_int64(0)
        best = None
        for rep in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            st = lib.hy3d_probe_mma_i8(n, 4000, sparse, ctypes.byref(ops), cur)
            e1.record()
            torch.cuda.synchronize()
            if st != 0:
                best = None
                break
            if rep:
                ms = e0.elapsed_time(e1)
                best = ms if best is None else min(best, ms)
        out[name] = round(ops.value / (best * 1e-3) / 1e12, 1) if best else None
    nbytes = 1 << 30
    a = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    b = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    for name, mode, moved in (("hbm_write_only_gbs", 0, nbytes), ("hbm_read_only_gbs", 1, nbytes),
                              ("hbm_copy_gbs", 2, 2 * nbytes)):
        best = None
        for rep in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            st = lib.hy3d_probe_hbm(mode, a.data_ptr(), b.data_ptr(), nbytes, cur)
            e1.record()
            torch.cuda.synchronize()
            if st != 0:
                best = None
                break
            if rep:
                ms = e0.elapsed_time(e1)
                best = ms if best is None else min(best, ms)
        out[name] = round(moved / (best * 1e-3) / 1e9, 1) if best else None
    del a, b
    torch.cuda.empty_cache()
    # tensor memory -> registers: 16 warps per SM, two tcgen05.ld 32x32b.x16 in flight per warp
    moved = ctypes.c_int64(0)
    best = None
    for rep in range(4):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        st = lib.hy3d_probe_tmem_ld(16, 2, 10000, ctypes.byref(moved), cur)
        e1.record()
        torch.cuda.synchronize()
        if st != 0:
            best = None
            break
        if rep:
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
    out["tmem_to_registers_tbs"] = round(moved.value / (best * 1e-3) / 1e12, 1) if best else None
    out["how"] = ("tcgen05.mma kind::i8 128x256x32 (sparse: 128x240x64) on resident operands, 4000 groups of 4 per SM, "
                  "best of 3; 1 GiB streams with 16-byte accesses from 592 CTAs, best of 3")
    return out


def per_shape_table(ctx: Ctx, shapes):
    """Per-shape device time (us) of the quantiser, the dense and sparse GEMMs, the whole dense
    layer, the same layer through the one-launch kernel where it takes the shape, cuBLAS bf16
    F.linear and the vendor INT8 GEMM, each replayed as a CUDA graph over rotating buffer sets
    larger than L2 (cold operands)."""
    lib, sp, dev = ctx.lib, ctx.sp, ctx.dev

    def graph_us(fns, reps=10):
        st = ctx.stream
        with torch.cuda.stream(st):
            for f in fns:
                f(st.cuda_stream)
            st.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for f in fns:
                    f(st.cuda_stream)
            for _ in range(3):
                g.replay()
            st.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for _ in range(reps):
                g.replay()
            e1.record(st)
            st.synchronize()
        return e0.elapsed_time(e1) / reps / len(fns) * 1e3

    def ck(st):
        if st != 0:
            raise RuntimeError(f"status {st}")

    rows = []
    for (M, K, N) in shapes:
        per_set = M * K * 3 + N * K + 2 * M * N
        R = max(2, min(16, int(300e6 // per_set) + 1))
        xs = [torch.randn(M, K, device=dev).bfloat16() for _ in range(R)]
        qs = [torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev) for _ in range(R)]
        ss = [torch.rand(M, device=dev) * 0.01 for _ in range(R)]
        ws = [torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(R)]
        wsc = torch.rand(N, device=dev).bfloat16()
        bias = torch.rand(N, device=dev).bfloat16()
        outs = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(R)]
        r = {"mkn": [M, K, N]}
        r["quant_us"] = graph_us([lambda s, i=i: ck(lib.hy3d_quantize_rows(
            xs[i].data_ptr(), 1, M, K, K, qs[i].data_ptr(), ss[i].data_ptr(), s)) for i in range(R)])
        r["gemm_dense_us"] = graph_us([lambda s, i=i: ck(lib.hy3d_gemm_w8a8_dense(
            qs[i].data_ptr(), ws[i].data_ptr(), ss[i].data_ptr(), wsc.data_ptr(), 1, bias.data_ptr(), 1,
            outs[i].data_ptr(), 1, M, N, K, 0, 0, 0, s)) for i in range(R)])
        import ctypes
        wsb = ctypes.c_int64(0)
        planned = lib.hy3d_dense_splitk_plan(M, N, K, 0, ctypes.byref(wsb))
        if planned > 1:     # few rows, deep K: K ranges side by side + reduce / epilogue kernel
            part = torch.empty(wsb.value // 4, dtype=torch.int32, device=dev)
            r["gemm_dense_splitk_us"] = graph_us([lambda s, i=i: ck(lib.hy3d_gemm_w8a8_dense_splitk(
                qs[i].data_ptr(), ws[i].data_ptr(), ss[i].data_ptr(), wsc.data_ptr(), 1, bias.data_ptr(), 1,
                outs[i].data_ptr(), 1, M, N, K, 0, planned, part.data_ptr(), wsb.value, s)) for i in range(R)])
            r["splitk_ranges"] = planned
        r["layer_dense_us"] = graph_us([lambda s, i=i: ck(lib.hy3d_linear_w8a8_dense(
            xs[i].data_ptr(), 1, K, qs[i].data_ptr(), ss[i].data_ptr(), ws[i].data_ptr(), wsc.data_ptr(), 1,
            bias.data_ptr(), 1, outs[i].data_ptr(), 1, M, N, K, 0, 0, 0, s)) for i in range(R)])
        if K <= 1280 and K % 32 == 0:
            try:
                r["layer_one_launch_us"] = graph_us([lambda s, i=i: ck(lib.hy3d_linear_w8a8_dense_fused(
                    xs[i].data_ptr(), 1, K, None, ws[i].data_ptr(), wsc.data_ptr(), 1, bias.data_ptr(), 1,
                    outs[i].data_ptr(), 1, M, N, K, 0, 0, s)) for i in range(R)])
            except RuntimeError:
                r["layer_one_launch_us"] = None
        if K % 64 == 0:
            packs = [sp.sparse_prune_and_pack(w) for w in ws]
            r["gemm_sparse_us"] = graph_us([lambda s, i=i: ck(lib.hy3d_gemm_w8a8_sparse24(
                qs[i].data_ptr(), ss[i].data_ptr(), packs[i][0].data_ptr(), packs[i][1].data_ptr(),
                packs[i][1].shape[1], wsc.data_ptr(), 1, bias.data_ptr(), 1, outs[i].data_ptr(), 1, M, N, K, 0, 0, s))
                for i in range(R)])
            del packs
        wb = [w.bfloat16() for w in ws]
        r["bf16_linear_us"] = graph_us([lambda s, i=i: torch.nn.functional.linear(xs[i], wb[i], bias)
                                        for i in range(R)])
        if M > 32:
            try:
                r["vendor_int8_gemm_us"] = graph_us([lambda s, i=i: torch._int_mm(qs[i], ws[i].t()) for i in range(R)])
            except Exception:
                r["vendor_int8_gemm_us"] = None
        ops = 2.0 * M * K * N
        r["gemm_dense_tops"] = round(ops / r["gemm_dense_us"] / 1e6, 1)
        r["layer_dense_tops"] = round(ops / r["layer_dense_us"] / 1e6, 1)
        rows.append({k: (round(v, 2) if isinstance(v, float) else v) for k, v in r.items()})
        del xs, qs, ss, ws, outs, wb
        torch.cuda.empty_cache()
    return rows


def run_ref_kernels(args):
    """`--workload ref_kernels`: times the reference's own CUDA kernels, rebuilt for sm_100 by
    baseline/make_ref_kernels.py (only the -gencode target changed), on the sweep's shapes:
    `int8_linear_tc` (wmma dense, csrc/int8_gemm_tc.cu:312-320) and `sparse_int8_linear`
    (mma.sp, csrc/int8_sparse_tc.cu:2027-2044), fp16 in / out as they were written.  Runs in a
    process of its own (the main benchmark calls it as a child) and prints one JSON line."""
    if not torch.cuda.is_available():
        raise RuntimeError("needs a CUDA device")
    dev = torch.device("cuda", 0)
    out = {"how": "reference sources compiled with -O3 --use_fast_math -gencode=arch=compute_100,code=sm_100; "
                  "plain CUDA events over rotating buffer sets (its dense kernel launches on the legacy default "
                  "stream and cannot be graph-captured)", "rows": []}
    try:
        mk = importlib.import_module("baseline.make_ref_kernels")
        tcm, spm = mk.load_module("int8_gemm_tc"), mk.load_module("int8_sparse_tc")
    except Exception as e:   # noqa: BLE001
        print(json.dumps({"unavailable": f"{type(e).__name__}: {e}"}), flush=True)
        return
    if tcm is None and spm is None:
        print(json.dumps({"unavailable": "baseline/_ref holds no built extension (baseline/make_ref_kernels.py was not run)"}), flush=True)
        return

    def event_us(fn, R, reps=5):
        for i in range(R):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for i in range(R):
                fn(i)
        e1.record()
        torch.cuda.synchronize()
        return round(e0.elapsed_time(e1) / reps / R * 1e3, 2)

    for (M, K, N) in SWEEP:
        per_set = M * K * 3 + N * K + 2 * M * N
        R = max(2, min(16, int(300e6 // per_set) + 1))
        xh = [torch.randn(M, K, device=dev).half() for _ in range(R)]
        ws = [torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(R)]
        wsc = (torch.rand(N, device=dev) * 1e-3).half()
        bias = torch.rand(N, device=dev).half()
        r = {"mkn": [M, K, N]}
        if tcm is not None:
            try:
                r["reference_dense_layer_us"] = event_us(lambda i: tcm.int8_linear_tc(xh[i], ws[i], wsc, bias), R)
            except Exception as e:   # noqa: BLE001
                r["reference_dense_layer_us"] = f"error: {type(e).__name__}: {str(e)[:120]}"
        if spm is not None and K >= 640:
            try:
                packs = [spm.sparse_prune_and_pack(w) for w in ws]
                r["reference_sparse_layer_us"] = event_us(
                    lambda i: spm.sparse_int8_linear(xh[i], packs[i][0], packs[i][1], wsc, bias), R)
            except Exception as e:   # noqa: BLE001
                r["reference_sparse_layer_us"] = f"error: {type(e).__name__}: {str(e)[:120]}"
        out["rows"].append(r)
        del xh, ws
        torch.cuda.empty_cache()
    print(json.dumps(out), flush=True)


def reference_kernels_child():
    """Runs `--workload ref_kernels` as a child process (a fault in foreign kernels must not take
    the benchmark down) and returns its record."""
    import subprocess
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref")):
        return {"unavailable": "baseline/_ref is absent (baseline/make_ref_kernels.py was not run)"}
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--workload", "ref_kernels"],
                           capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
        for ln in reversed(r.stdout.strip().splitlines()):
            if ln.startswith("{"):
                return json.loads(ln)
        return {"unavailable": f"child exited {r.returncode}: {r.stderr.strip()[-300:]}"}
    except Exception as e:   # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"}


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------
def run_ours(args):
    ctx = Ctx()
    rank, world, dev = ctx.rank, ctx.world, ctx.dev
    sparse_headline = args.workload == "sparse_sweep"
    peaks = load_peaks()
    bf16_peak = peaks.get("bf16_tflops", 1590.0)
    hbm_gbs = peaks.get("hbm_gbs", 6650.0)
    peak_src = "measured (MEASURED_PEAKS.json)" if peaks else "fallback"

    sweep = Sweep(ctx, sparse_headline, 1000 * (rank + 1))
    g_step, g_gemm = sweep.graphs()
    sampler = ClockSampler(ctx.local_rank) if rank == 0 else None
    ms_runs = timed_repeats(ctx, g_step.replay, args.steps, args.warmup, repeats=args.repeats, sampler=sampler)
    ms_step = statistics.median(ms_runs)
    value = world * sweep.ops / (ms_step * 1e-3) / 1e12
    gemm_runs = timed_repeats(ctx, g_gemm.replay, args.steps, max(args.warmup, 3), repeats=3)
    ms_gemm = statistics.median(gemm_runs)
    gemm_tops = sweep.ops / (ms_gemm * 1e-3) / 1e12

    denoms = measured_denominators(ctx)
    sp_mult = 2.0 if sparse_headline else 1.0
    proxy_peak = 2.0 * bf16_peak * sp_mult
    measured_peak = denoms.get("int8_sparse24_tops" if sparse_headline else "int8_dense_tops")
    nominal_peak = 4500.0 * sp_mult

    def bounds(shapes, sparse, peak_tops, write_gbs=None):
        """Time a kernel sitting on both rooflines would need: per shape the larger of ops / tensor
        peak and algorithmic GEMM bytes / HBM rate (output bytes at the write-only rate if given)."""
        t, n_hbm = 0.0, 0
        per = []
        for (M, K, N) in shapes:
            w_bytes = N * K * (0.625 if sparse else 1.0)
            t_tc = 2.0 * M * K * N / (peak_tops * 1e12)
            rd = M * K + w_bytes + 4 * M + 4 * N
            wr = 2.0 * M * N
            t_mem = (rd + wr) / (hbm_gbs * 1e9) if not write_gbs else rd / (hbm_gbs * 1e9) + wr / (write_gbs * 1e9)
            t += max(t_tc, t_mem)
            n_hbm += 1 if t_mem > t_tc else 0
            per.append((t_tc, t_mem))
        return t, n_hbm, per

    peak_for_bound = measured_peak or proxy_peak
    t_bound, n_hbm_bound, _ = bounds(SWEEP, sparse_headline, peak_for_bound)
    roofline = {
        "bound": "tensor", "kernel": "gemm_sparse_kernel" if sparse_headline else "gemm_dense_kernel",
        "achieved": round(gemm_tops, 1), "peak": round(measured_peak or proxy_peak, 1), "unit": "TOP/s",
        "frac": round(gemm_tops / (measured_peak or proxy_peak), 4),
        "peak_source": ("of measured: resident-operand tcgen05.mma kind::i8 issue loop on this GPU in this run"
                        if measured_peak else f"of {peak_src}: 2 x bf16 burst"),
        "frac_of_2x_bf16_burst": round(gemm_tops / proxy_peak, 4), "peak_2x_bf16_burst": round(proxy_peak, 1),
        "frac_of_nominal": round(gemm_tops / nominal_peak, 4), "peak_nominal": nominal_peak,
        "traffic": TRAFFIC_BYTES_PER_LAUNCH["sparse" if sparse_headline else "dense"],
        "traffic_source": "ncu dram bytes of one launch (profiles/), scaled by the sweep's algorithmic bytes",
        "launches_per_step": len(SWEEP), "avg_launch_us": round(ms_gemm * 1e3 / len(SWEEP), 2),
        "per_shape_bound": {"ms_per_step_at_bound": round(t_bound * 1e3, 4),
                            "frac_of_bound": round(t_bound / (ms_gemm * 1e-3), 4),
                            "hbm_bound_shapes": n_hbm_bound, "shapes": len(SWEEP),
                            "note": "sum over shapes of max(ops / measured INT8 peak, algorithmic bytes / measured copy GB/s)"}}

    # End to end through the public module API with host buffers.
    e2e = None
    if not args.no_e2e:
        host_x = [x.cpu().pin_memory() for x in sweep.xs]
        host_y = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for M, K, N in sweep.raw]
        h2d = sum(t.numel() * t.element_size() for t in host_x)
        d2h = sum(t.numel() * t.element_size() for t in host_y)
        host_io = importlib.import_module(PKG + ".host_io")
        pipe = host_io.HostPipeline(dev)
        n_e2e = max(2, min(args.steps, 10))
        for _ in range(2):
            pipe.run(sweep.layers, host_x, host_y)
        torch.cuda.synchronize()
        ctx.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            pipe.run(sweep.layers, host_x, host_y)
        e1.record()
        torch.cuda.synchronize()
        ms = ctx.max_over_ranks(e0.elapsed_time(e1) / n_e2e)
        e2e = {"value": round(world * sweep.ops / (ms * 1e-3) / 1e12, 2), "unit": "TOPS",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(ms, 3),
               "steps": n_e2e,
               "note": "every rank's pinned-host copies share one host memory system / PCIe root: this number "
                       "does not scale with N" if world > 1 else None}
        del host_x, host_y

    line = {
        "metric": METRIC, "value": round(value, 2), "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "ms_per_step_spread": spread(ms_runs),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "s8*s8->s32, bf16 in/out", "data": "synthetic",
        "config": {"workload": ("2:4-sparse" if sparse_headline else "dense") +
                   " W8A8 linear sweep, 12 SD2.1 texture-UNet shapes (BASELINE configs[%d])" % (2 if sparse_headline else 1),
                   "shapes_mkn": SWEEP, "layer": "bf16 x -> per-token quantise -> INT8 GEMM -> rescale+bias -> bf16",
                   "l2": "inputs larger than L2: one step touches > 1 GB, graph replays back to back",
                   "timing": "CUDA-graph replay, CUDA events on the launching stream, max over ranks, "
                             "median of %d timed regions of --steps replays" % args.repeats},
        "roofline": roofline, "e2e": e2e,
        "gpu_launches": 2 * len(SWEEP) * args.steps * args.repeats,
        "gemm_only": {"ms_per_step": round(ms_gemm, 4), "tops": round(gemm_tops, 1), "spread_ms": spread(gemm_runs)},
        "measured_denominators": denoms, "env_knobs": env_knobs(),
    }

    if not args.quick:
        # ---- bf16 cuBLAS over the same twelve shapes: the yardstick an INT8 layer has to beat ----
        wb = [torch.empty((N, K), dtype=torch.bfloat16, device=dev).normal_(0, 0.02) for M, K, N in sweep.raw]
        bb = [L.bias for L in sweep.layers]

        def bf16_step(_s):
            for i in range(len(sweep.raw)):
                torch.nn.functional.linear(sweep.xs[i], wb[i], bb[i])
        g_bf16 = capture(ctx, bf16_step)
        bf16_runs = timed_repeats(ctx, g_bf16.replay, max(20, args.steps // 4), 3, repeats=3)
        line["bf16_linear_ms_per_step"] = round(statistics.median(bf16_runs), 4)
        line["layer_vs_bf16_cublas"] = round(statistics.median(bf16_runs) / ms_step, 3)
        del wb, g_bf16

        # ---- the other sweep (configs[2] when the headline is configs[1]) ----
        other = Sweep(ctx, not sparse_headline, 1000 * (rank + 1))
        og_step, og_gemm = other.graphs()
        o_runs = timed_repeats(ctx, og_step.replay, max(20, args.steps // 4), 3, repeats=3)
        og_runs = timed_repeats(ctx, og_gemm.replay, max(20, args.steps // 4), 3, repeats=3)
        o_ms, og_ms = statistics.median(o_runs), statistics.median(og_runs)
        o_peak = denoms.get("int8_dense_tops" if sparse_headline else "int8_sparse24_tops") or (proxy_peak / sp_mult * (1 if sparse_headline else 2))
        o_tops = other.ops / (og_ms * 1e-3) / 1e12
        line["dense" if sparse_headline else "sparse"] = {
            "config": "BASELINE configs[%d]" % (1 if sparse_headline else 2),
            "value": round(world * other.ops / (o_ms * 1e-3) / 1e12, 2), "unit": "TOPS (dense-equivalent)",
            "ms_per_step": round(o_ms, 4), "gemm_only_ms_per_step": round(og_ms, 4), "gemm_only_tops": round(o_tops, 1),
            "roofline": {"bound": "tensor", "achieved": round(o_tops, 1), "peak": round(o_peak, 1), "unit": "TOP/s",
                         "frac": round(o_tops / o_peak, 4), "peak_source": "of measured (probe of this run)"}}
        del other, og_step, og_gemm
        torch.cuda.empty_cache()

        # ---- token-split ("strong") form of the sweep: rank r takes rows [r*M/N, (r+1)*M/N) ----
        if world > 1:
            part = Sweep(ctx, sparse_headline, 1000, row_range=(rank / world, (rank + 1) / world))
            pg_step, _ = part.graphs()
            p_runs = timed_repeats(ctx, pg_step.replay, max(20, args.steps // 4), 3, repeats=3)
            p_ms = statistics.median(p_runs)
            line["strong"] = {"scaling": "strong", "split": "GEMM M (tokens): rows [r*M/N, (r+1)*M/N) per rank, weights replicated, no collective",
                              "value": round(sweep_ops() / (p_ms * 1e-3) / 1e12, 2), "unit": "TOPS",
                              "ms_per_step": round(p_ms, 4)}
            del part, pg_step
            torch.cuda.empty_cache()

        # ---- per-shape table (rank 0's GPU only; the other ranks idle meanwhile) ----
        if rank == 0:
            rows = per_shape_table(ctx, SWEEP + (DINO_SHAPES if world == 1 else []))
            line["per_shape_us"] = rows
            if world == 1:
                line["reference_kernels_us"] = reference_kernels_child()
            wr = denoms.get("hbm_write_only_gbs")
            targets = []
            for r in rows[:3]:
                M, K, N = r["mkn"]
                t_tc = 2.0 * M * K * N / ((measured_peak or proxy_peak) * 1e12) * 1e6
                rd, wrb = M * K + N * K + 4 * M + 4 * N, 2.0 * M * N
                t_hbm = (rd + wrb) / (hbm_gbs * 1e9) * 1e6
                t_hbm_w = (rd / (hbm_gbs * 1e9) + wrb / (wr * 1e9)) * 1e6 if wr else None
                targets.append({"mkn": r["mkn"], "gemm_us": r["gemm_dense_us"],
                                "tops_over_tensor_peak": round(r["gemm_dense_tops"] / (measured_peak or proxy_peak), 3),
                                "tops_over_nominal_4500": round(r["gemm_dense_tops"] / 4500.0, 3),
                                "achieved_over_hbm_bound_copy_rate": round(max(t_tc, t_hbm) / r["gemm_dense_us"], 3),
                                "achieved_over_hbm_bound_write_rate": round(max(t_tc, t_hbm_w) / r["gemm_dense_us"], 3) if t_hbm_w else None})
            line["north_star_49152_token_shapes"] = targets
        ctx.barrier()

        # ---- UNet step (configs[3]) and multi-mesh batch (configs[4]) ----
        del sweep, g_step, g_gemm
        torch.cuda.empty_cache()
        try:
            line["unet"] = unet_record(ctx, args)
            line["multimesh"] = multimesh_record(ctx, args)
        except Exception as e:   # noqa: BLE001 - the headline line is still printed
            line["unet_error"] = f"{type(e).__name__}: {e}"

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu_baseline = cpu_reference(steps=3, warmup=1, frac=args.cpu_frac)["cpu_baseline"]
    line["cpu_baseline"] = cpu_baseline
    line["clocks"] = sampler.summary() if sampler else None

    status = ctx.tc.device_status()
    if status != 0:
        raise RuntimeError(f"a kernel reported device status {status}")
    if rank == 0:
        print(json.dumps(line), flush=True)
    ctx.close()


# ---------------------------------------------------------------------------------------
# UNet denoise (BASELINE configs[3]) and multi-mesh batch (configs[4])
# ---------------------------------------------------------------------------------------
def unet_record(ctx: Ctx, args):
    """ms per denoise step (CUDA-graph replay of the 12-sample forward) with dense INT8, mixed
    dense / 2:4-sparse INT8 and unquantised bf16 linears."""
    mm = importlib.import_module(PKG + ".multimesh")
    out = {"config": "BASELINE configs[3]: SD2.1-architecture UNet, 2 (CFG) x 6 views x 64x64x4 latents, "
                     "multiview attention, random init", "unit": "ms/step", "steps": 20}
    # "none": the stock PyTorch model (bf16 linears, torch GroupNorm); "none_nhwc_groupnorm": the
    # same with this library's channels-last GroupNorm kernel, so that the INT8 linears' own
    # contribution can be read off as (none_nhwc_groupnorm - dense); "mixed_torch_groupnorm":
    # the INT8 model with torch's GroupNorm.
    variants = (("dense", "dense", None), ("mixed", "mixed", None), ("none", "none", False),
                ("none_nhwc_groupnorm", "none", True), ("mixed_torch_groupnorm", "mixed", False))
    for key, quant, fused_gn in variants:
        unet, stats = mm.build_texture_unet(ctx.dev, torch.bfloat16, quant, seed=0, init_on_device=True,
                                            fused_gn=fused_gn)
        step = mm.GraphedStep(unet, 12, 64, 77, 1024, torch.bfloat16, ctx.dev)
        runs = timed_repeats(ctx, step.graph.replay, 20, 3, repeats=3)
        out[key] = round(statistics.median(runs), 3)
        if key == "mixed":
            out["mixed_layers"] = {k: v for k, v in stats.items() if isinstance(v, int)}
            ctx._unet_mixed = unet        # reused by the multi-mesh record
        else:
            del unet
        del step
        torch.cuda.empty_cache()
    return out


def multimesh_record(ctx: Ctx, args):
    """32 meshes x 10 INT8 denoise steps, seeds 0..31 sharded round-robin over the ranks, bf16
    latents gathered on rank 0 with one NCCL gather; device time by CUDA events, max over ranks."""
    mm = importlib.import_module(PKG + ".multimesh")
    unet = getattr(ctx, "_unet_mixed", None)
    if unet is None:
        unet, _ = mm.build_texture_unet(ctx.dev, torch.bfloat16, "mixed", seed=0, init_on_device=True)
    seeds = list(range(32))
    mine = mm.partition(seeds, ctx.rank, ctx.world)
    inputs = mm.prefetch_mesh_inputs(mine)
    # warm-up: builds the captured step and the gather's connections (first use of a NCCL
    # point-to-point path sets up its channels, hundreds of ms that belong to no mesh)
    warm, _ = mm.denoise_meshes(unet, mine[:1], device=ctx.dev, inputs=inputs)
    mm.gather_results(warm, [mm.partition(seeds, r, ctx.world)[0] for r in range(ctx.world)],
                      (6, 4, 64, 64), torch.bfloat16, ctx.dev, dst=0)
    del warm
    ctx.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    local, _ = mm.denoise_meshes(unet, mine, device=ctx.dev, inputs=inputs)
    results, missing = mm.gather_results(local, seeds, (6, 4, 64, 64), torch.bfloat16, ctx.dev, dst=0)
    e1.record()
    torch.cuda.synchronize()
    sec = ctx.max_over_ranks(e0.elapsed_time(e1)) * 1e-3
    del ctx._unet_mixed
    return {"config": "BASELINE configs[4]: 32 meshes x 10 denoise steps, mixed INT8 UNet", "value": round(32 / sec, 3),
            "unit": "meshes/s", "n_gpus": ctx.world, "scaling": "strong", "seconds": round(sec, 3),
            "ms_per_step_per_rank": round(sec * 1e3 / (10 * len(mine)), 3),
            "collected": len(results) if results is not None else None, "missing": missing,
            "h2d_bytes_per_mesh": int((6 * 4 * 64 * 64 + 2 * 6 * 77 * 1024) * 2), "d2h_bytes_per_mesh": 0}


def run_unet(args):
    """`--workload unet` / `multimesh`: the sub-records above as lines of their own."""
    ctx = Ctx()
    if args.workload == "unet":
        rec = unet_record(ctx, args)
        line = {"metric": "UNet denoise ms/step (6 views)", "value": rec[args.quant if args.quant in rec else "mixed"],
                "unit": "ms", "n_gpus": ctx.world, "steps": 20, "warmup": 3, "higher_is_better": False,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16 + W8A8 linears", "data": "synthetic",
                "config": {"workload": rec["config"], "quant": args.quant}, "unet": rec, "env_knobs": env_knobs()}
    else:
        rec = multimesh_record(ctx, args)
        line = {"metric": "multi-mesh texture batch, meshes/s", "value": rec["value"], "unit": "meshes/s",
                "n_gpus": ctx.world, "steps": 10, "warmup": 1, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16 + W8A8 linears", "data": "synthetic",
                "config": {"workload": rec["config"]}, "multimesh": rec, "env_knobs": env_knobs()}
    if ctx.rank == 0:
        print(json.dumps(line), flush=True)
    ctx.close()


def run_one_shape(args):
    """Runs one entry point `--launches` times on one shape (synthetic operands) and checks the
    status codes.  Nothing is timed here: a profiler does that."""
    ctx = Ctx()
    lib, sp, dev = ctx.lib, ctx.sp, "cuda"
    if args.kernel == "unet":
        # `--launches` eager (un-graphed) forward passes of the full-size UNet of configs[3], so
        # that a profiler's launch list shows every kernel of a denoise step by name.
        mm = importlib.import_module(PKG + ".multimesh")
        unet, _ = mm.build_texture_unet(dev, torch.bfloat16, args.quant, seed=0, init_on_device=True,
                                        fused_gn=False if args.torch_groupnorm else None)
        lat, cond, uncond = mm.mesh_inputs(0, device=dev)
        x = torch.cat([lat, lat]); c = torch.cat([uncond, cond])
        t = torch.full((12,), 500, device=dev)
        with torch.no_grad():
            for _ in range(args.launches):
                unet(x, t, c)
        torch.cuda.synchronize()
        if ctx.tc.device_status() != 0:
            raise SystemExit("device status non-zero")
        print("ok")
        ctx.close()
        return
    M, K, N = (int(v) for v in args.shape.split("x"))
    if args.kernel == "groupnorm":
        # --shape is B x (H*W) x C here: GroupNorm + SiLU over a channels-last activation
        B, HW, C = M, K, N
        side = int(round(HW ** 0.5))
        xg = torch.randn(B, C, side, HW // side, device=dev).bfloat16().contiguous(memory_format=torch.channels_last)
        gam, bet = torch.randn(C, device=dev).bfloat16(), torch.randn(C, device=dev).bfloat16()
        ik = importlib.import_module(PKG + ".csrc.build").load_int8_kernels()
        ws = torch.empty(1 << 16, dtype=torch.float32, device=dev)
        yg = torch.empty_like(xg, memory_format=torch.channels_last)
        for _ in range(args.launches):
            ik.groupnorm_nhwc(xg, 32, gam, bet, 1e-5, silu=True, out=yg, workspace=ws)
        torch.cuda.synchronize()
        print("ok")
        ctx.close()
        return
    x = torch.randn(M, K, device=dev).bfloat16()
    q = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev)
    s = torch.rand(M, device=dev) * 0.01
    w = torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev)
    ws = torch.rand(N, device=dev).bfloat16()
    b = torch.rand(N, device=dev).bfloat16()
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    st = torch.cuda.current_stream().cuda_stream
    kind = args.kernel
    if kind == "sparse":
        comp, meta = sp.sparse_prune_and_pack(w)
    if kind == "prune":
        comp = torch.empty(N, K // 2, dtype=torch.int8, device=dev)
        ld = 4 * ((K + 127) // 128)
        meta = torch.empty(N, ld, dtype=torch.int32, device=dev)
    for _ in range(args.launches):
        if kind == "dense":
            r = lib.hy3d_gemm_w8a8_dense(q.data_ptr(), w.data_ptr(), s.data_ptr(), ws.data_ptr(), 1,
                                         b.data_ptr(), 1, out.data_ptr(), 1, M, N, K, 0, 0, 0, st)
        elif kind == "sparse":
            r = lib.hy3d_gemm_w8a8_sparse24(q.data_ptr(), s.data_ptr(), comp.data_ptr(), meta.data_ptr(),
                                            meta.shape[1], ws.data_ptr(), 1, b.data_ptr(), 1,
                                            out.data_ptr(), 1, M, N, K, 0, 0, st)
        elif kind == "quant":
            r = lib.hy3d_quantize_rows(x.data_ptr(), 1, M, K, K, q.data_ptr(), s.data_ptr(), st)
        elif kind == "lnquant":
            r = lib.hy3d_layernorm_quantize(x.data_ptr(), 1, M, K, K, ws.data_ptr() if N == K else None,
                                            b.data_ptr() if N == K else None, 1, 1e-5, q.data_ptr(),
                                            s.data_ptr(), None, st)
        elif kind == "prune":
            r = lib.hy3d_prune_pack_24(w.data_ptr(), N, K, comp.data_ptr(), None, meta.data_ptr(), ld, st)
        elif kind == "fused":
            r = lib.hy3d_linear_w8a8_dense_fused(x.data_ptr(), 1, K, None, w.data_ptr(), ws.data_ptr(), 1,
                                                 b.data_ptr(), 1, out.data_ptr(), 1, M, N, K, 0, 0, st)
        else:
            raise SystemExit(f"unknown kernel {kind!r}")
        if r != 0:
            raise SystemExit(f"status {r}")
    torch.cuda.synchronize()
    if ctx.tc.device_status() != 0:
        raise SystemExit("device status non-zero")
    print("ok")
    ctx.close()


# ---------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CPU W8A8 path
# ---------------------------------------------------------------------------------------
def cpu_reference(steps, warmup, frac):
    """Times the reference's CPU implementation of the layer -- `Int8Linear.from_linear(...)`,
    then `_forward_int_mm(x, M) + bias` (per-token quantise, torch._int_mm, fp32 rescale; the
    reference's quantize_utils.py:203-223, 293-309, 339-345) -- on a row sample of every sweep
    shape, with all host threads.  The module itself is used when oracle/make_ref.py has placed a
    copy under oracle/_ref/ (kind "reference"); otherwise the restatement in oracle/oracle.py
    (kind "port", with the reason)."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    ref, why = None, None
    try:
        mk = importlib.import_module("oracle.make_ref")
        ref = mk.load()
        if ref is None:
            why = "oracle/_ref/quantize_utils.py is absent (oracle/make_ref.py was not run)"
    except Exception as e:   # noqa: BLE001
        why = f"reference module failed to import: {type(e).__name__}: {e}"
    from oracle import oracle as O     # checker / baseline only -- never on the product path
    cases = []
    for i, (M, K, N) in enumerate(SWEEP):
        rows = max(32, int(M * frac))
        g = torch.Generator().manual_seed(1000 + i)
        x = torch.randn(rows, K, generator=g)
        mask = torch.rand(rows, K, generator=g) < 0.001
        x = torch.where(mask, torch.full_like(x, 20.0), x)
        w = (torch.randn(N, K, generator=g) * 0.02)
        b = (torch.randn(N, generator=g) * 0.01)
        if ref is not None:
            lin = torch.nn.Linear(K, N)
            lin.weight.data.copy_(w)
            lin.bias.data.copy_(b)
            layer = ref.Int8Linear.from_linear(lin.half())
            cases.append((x.half(), layer, rows, K, N))
        else:
            wq, ws = O.quantize_weight(w.bfloat16())
            cases.append((x.bfloat16(), (wq, ws.bfloat16(), b.bfloat16()), rows, K, N))
    ops = sum(2.0 * r * k * n for _, _, r, k, n in cases)

    def step():
        for x, layer, rows, *_ in cases:
            if ref is not None:
                layer._forward_int_mm(x, rows) + layer.bias
            else:
                O.linear_w8a8(x, *layer)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    tops = ops / dt / 1e12
    sample = f"{frac:g} of the rows of each of the 12 sweep shapes (min 32), {steps} timed pass(es)"
    cb = {"value": round(tops, 4), "unit": "TOPS", "cores": threads, "kind": "reference" if ref is not None else "port",
          "sample": sample,
          "what": "Int8Linear._forward_int_mm + bias of the reference's quantize_utils.py on CPU tensors"
                  if ref is not None else "oracle.linear_w8a8 (restatement of the same path): " + str(why)}
    return {"tops": tops, "ms_per_step": dt * 1e3, "cpu_baseline": cb}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = cpu_reference(args.steps, args.warmup, args.cpu_frac)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(r["tops"], 4), "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(r["ms_per_step"], 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "s8*s8->s32, bf16 in/out", "data": "synthetic",
        "config": {"workload": "dense W8A8 linear sweep, 12 SD2.1 texture-UNet shapes (BASELINE configs[1])",
                   "shapes_mkn": SWEEP, "layer": "bf16 x -> per-token quantise -> INT8 GEMM -> rescale+bias -> bf16",
                   "l2": "host arm: no GPU", "timing": "host wall clock on rank 0, all host threads"},
        "cpu_baseline": r["cpu_baseline"],
        "e2e": {"value": round(r["tops"], 4), "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps per region (default: 200 sweep passes, 5 CPU reference passes)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps replays; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense_sweep",
                    choices=["dense_sweep", "sparse_sweep", "unet", "multimesh", "one_shape", "ref_kernels"])
    ap.add_argument("--quant", default="mixed", choices=["mixed", "dense", "sparse", "none"])
    ap.add_argument("--quick", action="store_true", help="headline, roofline and e2e only: no sub-records")
    ap.add_argument("--kernel", default="dense", help="one_shape: dense | sparse | quant | lnquant | prune | fused | groupnorm (shape = B x HW x C) | unet (eager UNet forwards)")
    ap.add_argument("--shape", default="8192x1280x1280", help="one_shape: MxKxN")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--torch-groupnorm", action="store_true",
                    help="one_shape --kernel unet: keep torch's GroupNorm / SiLU ops instead of the channels-last kernel")
    ap.add_argument("--cpu-frac", type=float, default=None,
                    help="row fraction of each shape timed on the CPU (default: all rows, fewer when "
                         "the requested number of reference passes would take more than ~2 minutes)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.steps is None:
        args.steps = 5 if args.impl == "reference" else 200
    if args.cpu_frac is None:
        # One pass over all rows takes ~0.6 s on the host cores of the GPU box.
        args.cpu_frac = 1.0
        if args.impl == "reference":
            args.cpu_frac = min(1.0, 120.0 / (0.6 * (args.steps + args.warmup)))
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "one_shape":
        run_one_shape(args)
    elif args.workload == "ref_kernels":
        run_ref_kernels(args)
    elif args.workload in ("unet", "multimesh"):
        run_unet(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
