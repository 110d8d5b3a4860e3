#!/usr/bin/env python
"""Benchmark of the W8A8 linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload dense_sweep|sparse_sweep|unet|multimesh] [--quant mixed|dense|sparse|none]

One "step" is one pass over the twelve SD2.1-style texture-UNet linear shapes (M = 2 x 6 views x
tokens per level: 49152 / 12288 / 3072 rows, plus the three cross-attention K/V shapes at
M = 12 x 77): for every shape a whole linear layer, bf16 activations in, per-token quantise,
INT8 tensor-core GEMM, rescale + bias, bf16 out.  Inputs are seeded synthetic tensors with the
configuration's shapes and value distributions (N(0,1) activations with 0.1 % outliers at
20 sigma, N(0,0.02) weights).  `value` is dense-equivalent TOPS (2*M*K*N per layer, summed over
the sweep and over ranks, divided by the slowest rank's time).

With N > 1 every rank runs the sweep on its own (differently seeded) activations -- the tokens
of a different mesh -- with replicated weights and no collective on the data path, so per-GPU
work is fixed ("weak" scaling).

The timed region replays a CUDA graph of one step; the sweep touches > 1 GB per step, so no
operand survives in the 126 MB L2 from one step to the next.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SWEEP = [
    (49152, 320, 320), (49152, 320, 2560), (49152, 1280, 320),
    (12288, 640, 640), (12288, 640, 5120), (12288, 2560, 640),
    (3072, 1280, 1280), (3072, 1280, 10240), (3072, 5120, 1280),
    (924, 1024, 320), (924, 1024, 640), (924, 1024, 1280),
]
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

    def summary(self, in_region):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s), "samples_in_timed_region": in_region,
                "power_w_max": max(self.power) if self.power else None}


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------
def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    qu = importlib.import_module("hunyuan3d-tools_b200.quantize_utils")
    build = importlib.import_module("hunyuan3d-tools_b200.csrc.build")
    tc = build.load_tc_gemm()
    sp = build.load_sparse_tc()
    sparse = args.workload == "sparse_sweep"

    layers, xs, raw = [], [], []
    for i, (M, K, N) in enumerate(SWEEP):
        x, w, b = make_inputs(i, M, K, N, 1000 * (rank + 1), dev)
        lin = torch.nn.Linear(K, N, device=dev, dtype=torch.bfloat16)
        lin.weight.data.copy_(w)
        lin.bias.data.copy_(b)
        layer = (qu.Int8Linear.from_linear_sparse if sparse else qu.Int8Linear.from_linear)(lin)
        layers.append(layer)
        xs.append(x)
        raw.append((M, K, N))
    ops_step = sweep_ops()

    # Pre-allocated workspaces / outputs so that a step is pure kernel launches through the
    # C ABI (the same entry points Int8Linear.forward uses).
    lib = tc._lib
    qs = [torch.empty((M, K), dtype=torch.int8, device=dev) for M, K, N in raw]
    ss = [torch.empty((M,), dtype=torch.float32, device=dev) for M, K, N in raw]
    outs = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for M, K, N in raw]

    def launch_linear(i, stream):
        M, K, N = raw[i]
        L = layers[i]
        if sparse:
            st = lib.hy3d_linear_w8a8_sparse24(
                xs[i].data_ptr(), 1, K, qs[i].data_ptr(), ss[i].data_ptr(),
                L.weight_sparse_comp.data_ptr(), L.weight_sparse_meta.data_ptr(),
                L.weight_sparse_meta.shape[1], L.weight_scale.data_ptr(), 1, L.bias.data_ptr(), 1,
                outs[i].data_ptr(), 1, M, N, K, 0, 0, stream)
        else:
            st = lib.hy3d_linear_w8a8_dense(
                xs[i].data_ptr(), 1, K, qs[i].data_ptr(), ss[i].data_ptr(),
                L.weight_int8_nk.data_ptr(), L.weight_scale.data_ptr(), 1, L.bias.data_ptr(), 1,
                outs[i].data_ptr(), 1, M, N, K, 0, 0, 0, stream)
        if st != 0:
            raise RuntimeError(f"linear launch failed with status {st}")

    def launch_gemm_only(i, stream):
        M, K, N = raw[i]
        L = layers[i]
        if sparse:
            st = lib.hy3d_gemm_w8a8_sparse24(
                qs[i].data_ptr(), ss[i].data_ptr(), L.weight_sparse_comp.data_ptr(),
                L.weight_sparse_meta.data_ptr(), L.weight_sparse_meta.shape[1],
                L.weight_scale.data_ptr(), 1, L.bias.data_ptr(), 1, outs[i].data_ptr(), 1, M, N, K,
                0, 0, stream)
        else:
            st = lib.hy3d_gemm_w8a8_dense(
                qs[i].data_ptr(), L.weight_int8_nk.data_ptr(), ss[i].data_ptr(),
                L.weight_scale.data_ptr(), 1, L.bias.data_ptr(), 1, outs[i].data_ptr(), 1, M, N, K,
                0, 0, 0, stream)
        if st != 0:
            raise RuntimeError(f"gemm launch failed with status {st}")

    stream = torch.cuda.Stream(device=dev)

    def capture(fn):
        with torch.cuda.stream(stream):
            fn(stream.cuda_stream)                       # first call outside capture (lazy set-up)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn(stream.cuda_stream)
        return g

    g_step = capture(lambda s: [launch_linear(i, s) for i in range(len(SWEEP))])
    g_gemm = capture(lambda s: [launch_gemm_only(i, s) for i in range(len(SWEEP))])

    def timed(graph, steps, warmup, sampler=None):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                graph.replay()
            stream.synchronize()
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if sampler:
                sampler.start()
            e0.record(stream)
            for _ in range(steps):
                graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            n_in = len(sampler.samples) if sampler else 0
            if sampler and n_in < 8:
                # The timed region was too short for the NVML poller: keep the same load
                # running (untimed) until a few samples exist.
                t_end = time.time() + 0.4
                while time.time() < t_end:
                    graph.replay()
                stream.synchronize()
            if sampler:
                sampler.stop()
            if dist is not None:
                dist.barrier()
            ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, n_in

    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms_total, n_in = timed(g_step, args.steps, args.warmup, sampler)
    ms_step = ms_total / args.steps
    value = world * ops_step / (ms_step * 1e-3) / 1e12

    # Dominant kernel (the GEMM) timed alone over the same sweep, same method.
    ms_gemm_total, _ = timed(g_gemm, args.steps, max(args.warmup, 3))
    ms_gemm = ms_gemm_total / args.steps
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    bf16_peak = peaks.get("bf16_tflops", 1590.0)
    peak_src = "2 x measured bf16 burst (MEASURED_PEAKS.json)" if peaks else "2 x fallback bf16 1590"
    int8_peak = 2.0 * bf16_peak * (2.0 if sparse else 1.0)
    gemm_tops = ops_step / (ms_gemm * 1e-3) / 1e12
    # Context for the fraction: what the vendor library's INT8 GEMM reaches on this GPU on a
    # large square problem (a library call, used only as a yardstick, never on the product path).
    lib_int8 = None
    try:
        a8 = torch.randint(-128, 128, (8192, 8192), dtype=torch.int8, device=dev)
        b8 = torch.randint(-128, 128, (8192, 8192), dtype=torch.int8, device=dev)
        for _ in range(2):
            torch._int_mm(a8, b8.t())
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch._int_mm(a8, b8.t()); e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        lib_int8 = round(2 * 8192 ** 3 / (best * 1e-3) / 1e12, 1)
    except Exception:
        pass
    # The same square problem through this library's GEMM (int8 in, bf16 out with the fused
    # rescale + bias epilogue): how close the kernel itself gets to the tensor roofline when the
    # shape lets it (the sweep's UNet shapes are mostly bound by HBM or by their short K).
    own_int8 = None
    if not sparse:
        try:
            n8 = 8192
            as8 = torch.rand(n8, device=dev) * 0.01
            ws8 = torch.rand(n8, device=dev).bfloat16()
            o8 = torch.empty((n8, n8), dtype=torch.bfloat16, device=dev)
            cur = torch.cuda.current_stream().cuda_stream
            best = 1e9
            for i in range(6):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                st = lib.hy3d_gemm_w8a8_dense(a8.data_ptr(), b8.data_ptr(), as8.data_ptr(), ws8.data_ptr(), 1,
                                              None, 1, o8.data_ptr(), 1, n8, n8, n8, 0, 0, 0, cur)
                e1.record()
                torch.cuda.synchronize()
                if st != 0:
                    raise RuntimeError(f"status {st}")
                if i:
                    best = min(best, e0.elapsed_time(e1))
            own_int8 = round(2 * n8 ** 3 / (best * 1e-3) / 1e12, 1)
            del as8, ws8, o8
        except Exception:
            pass
    try:
        del a8, b8
    except Exception:
        pass
    # The sweep mixes tensor-bound and HBM-bound shapes: sum over shapes of the larger of
    # (ops / tensor peak) and (algorithmic GEMM bytes / measured copy bandwidth) is the time
    # a kernel sitting on both rooflines would need for the same step.
    hbm_gbs = peaks.get("hbm_gbs", 6650.0)
    t_bound = 0.0
    n_hbm_bound = 0
    for (M, K, N) in SWEEP:
        w_bytes = N * K * (0.625 if sparse else 1.0)
        t_tc = 2.0 * M * K * N / (int8_peak * 1e12)
        t_mem = (M * K + w_bytes + 4 * M + 4 * N + 2 * M * N) / (hbm_gbs * 1e9)
        t_bound += max(t_tc, t_mem)
        n_hbm_bound += 1 if t_mem > t_tc else 0
    roofline = {"bound": "tensor", "kernel": "gemm_sparse_kernel" if sparse else "gemm_dense_kernel",
                "achieved": round(gemm_tops, 1), "peak": round(int8_peak, 1), "unit": "TOP/s",
                "frac": round(gemm_tops / int8_peak, 4), "peak_source": peak_src,
                "traffic": TRAFFIC_BYTES_PER_LAUNCH["sparse" if sparse else "dense"],
                "traffic_source": "ncu dram bytes of one launch (profiles/), scaled by the sweep's algorithmic bytes",
                "library_int8_gemm_8192_tops": lib_int8, "own_gemm_8192_tops": own_int8,
                "launches_per_step": len(SWEEP), "avg_launch_us": round(ms_gemm * 1e3 / len(SWEEP), 2),
                "per_shape_bound": {"ms_per_step_at_bound": round(t_bound * 1e3, 4),
                                    "frac_of_bound": round(t_bound / (ms_gemm * 1e-3), 4),
                                    "hbm_bound_shapes": n_hbm_bound, "shapes": len(SWEEP),
                                    "note": "sum over shapes of max(ops / peak, algorithmic bytes / measured copy GB/s)"}}

    # End to end through the public module API with host buffers.
    e2e = None
    if not args.no_e2e:
        host_x = [x.cpu().pin_memory() for x in xs]
        host_y = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for M, K, N in raw]
        h2d = sum(t.numel() * t.element_size() for t in host_x)
        d2h = sum(t.numel() * t.element_size() for t in host_y)

        host_io = importlib.import_module("hunyuan3d-tools_b200.host_io")
        pipe = host_io.HostPipeline(dev)

        def e2e_step():
            # Public module API on pinned host tensors; uploads, kernels and downloads of
            # neighbouring layers overlap on three streams (every byte still crosses PCIe).
            pipe.run(layers, host_x, host_y)

        n_e2e = max(2, min(args.steps, 10))
        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n_e2e
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        e2e = {"value": round(world * ops_step / (ms * 1e-3) / 1e12, 2), "unit": "TOPS",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(ms, 3),
               "steps": n_e2e}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu_baseline = cpu_reference(steps=3, warmup=1, frac=args.cpu_frac)["cpu_baseline"]

    status = tc.device_status()
    if status != 0:
        raise RuntimeError(f"a kernel reported device status {status}")

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "s8*s8->s32, bf16 in/out", "data": "synthetic",
            "config": {"workload": ("2:4-sparse" if sparse else "dense") +
                       " W8A8 linear sweep, 12 SD2.1 texture-UNet shapes (BASELINE configs[%d])" % (2 if sparse else 1),
                       "shapes_mkn": SWEEP, "layer": "bf16 x -> per-token quantise -> INT8 GEMM -> rescale+bias -> bf16",
                       "l2": "inputs larger than L2: one step touches > 1 GB, graph replays back to back",
                       "timing": "CUDA-graph replay, CUDA events on the launching stream, max over ranks"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": 2 * len(SWEEP) * args.steps,
            "clocks": sampler.summary(n_in) if sampler else None,
            "gemm_only": {"ms_per_step": round(ms_gemm, 4), "tops": round(gemm_tops, 1)},
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU W8A8 path, restated in oracle/
# ---------------------------------------------------------------------------------------
def cpu_reference(steps, warmup, frac):
    """Times the CPU restatement of the reference's W8A8 layer (its `_forward_int_mm` + bias:
    per-token quantise, torch._int_mm, fp32 rescale) on a row sample of every sweep shape."""
    from oracle import oracle as O     # checker / baseline only -- never on the product path
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    cases = []
    for i, (M, K, N) in enumerate(SWEEP):
        rows = max(32, int(M * frac))
        g = torch.Generator().manual_seed(1000 + i)
        x = torch.randn(rows, K, generator=g).bfloat16()
        w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
        b = (torch.randn(N, generator=g) * 0.01).bfloat16()
        wq, ws = O.quantize_weight(w)
        cases.append((x, wq, ws.bfloat16(), b, rows, K, N))
    ops = sum(2.0 * r * k * n for _, _, _, _, r, k, n in cases)

    def step():
        for x, wq, ws, b, *_ in cases:
            O.linear_w8a8(x, wq, ws, b)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    tops = ops / dt / 1e12
    sample = f"{frac:g} of the rows of each of the 12 sweep shapes (min 32), {steps} timed pass(es)"
    return {"tops": tops, "ms_per_step": dt * 1e3,
            "cpu_baseline": {"value": round(tops, 4), "unit": "TOPS", "cores": threads, "kind": "port",
                             "sample": sample}}


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
                   "shapes_mkn": SWEEP,
                   "note": "CPU restatement of the reference's quantize_utils W8A8 path (the reference is "
                           "Python and is not present on the GPU box); runs on rank 0 host cores only"},
        "cpu_baseline": r["cpu_baseline"],
        "e2e": {"value": round(r["tops"], 4), "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------
# UNet denoise (BASELINE configs[3]) and multi-mesh batch (configs[4])
# ---------------------------------------------------------------------------------------
def run_unet(args):
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    mm = importlib.import_module("hunyuan3d-tools_b200.multimesh")
    un = importlib.import_module("hunyuan3d-tools_b200.unet")
    unet, stats = mm.build_texture_unet(dev, torch.bfloat16, args.quant, seed=0)
    step = mm.GraphedStep(unet, 12, 64, 77, 1024, torch.bfloat16, dev)

    def sync_max(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.workload == "unet":
        for _ in range(args.warmup):
            step.graph.replay()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        sampler = ClockSampler(local_rank) if rank == 0 else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler:
            sampler.start()
        e0.record()
        for _ in range(args.steps):
            step.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.stop()
        ms_step = sync_max(e0.elapsed_time(e1) / args.steps)
        # end to end: host latents / context in, 10-step loop, host latents out
        lat, cond, uncond = mm.mesh_inputs(1000 + rank)
        lat, cond, uncond = lat.pin_memory(), cond.pin_memory(), uncond.pin_memory()
        host_out = torch.empty_like(lat).pin_memory()
        torch.cuda.synchronize()
        e0.record()
        out = un.denoise(unet, lat.to(dev, non_blocking=True), cond.to(dev, non_blocking=True),
                         uncond.to(dev, non_blocking=True), steps=10, step_fn=step)
        host_out.copy_(out, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = sync_max(e0.elapsed_time(e1) / 10)
        if rank == 0:
            print(json.dumps({
                "metric": "UNet denoise ms/step (6 views)", "value": round(ms_step, 3), "unit": "ms",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 3),
                "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 + W8A8 linears",
                "data": "synthetic",
                "config": {"workload": "one denoise step of the random-init SD2.1-architecture UNet, 2 (CFG) x 6 views "
                                       "x 64x64x4 latents, multiview attention (BASELINE configs[3])",
                           "quant": args.quant, "layers": stats,
                           "timing": "CUDA-graph replay of the 12-sample forward, one mesh per rank"},
                "e2e": {"value": round(e2e_ms, 3), "unit": "ms", "h2d_bytes_per_step": int((lat.numel() + 2 * cond.numel()) * 2 / 10),
                        "d2h_bytes_per_step": int(lat.numel() * 2 / 10)},
                "meshes_per_s": round(world / (10 * ms_step * 1e-3), 2),
                "clocks": sampler.summary(len(sampler.samples)) if sampler else None,
            }), flush=True)
    else:   # multimesh: 32 meshes sharded over the ranks, latents gathered on rank 0
        seeds = list(range(32))
        mine = mm.partition(seeds, rank, world)
        mm.denoise_meshes(unet, mine[:1], device=dev)           # warm-up
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        local, _ = mm.denoise_meshes(unet, mine, device=dev)
        results, missing = mm.gather_results(local, seeds, (6, 4, 64, 64), torch.bfloat16, dev, dst=0)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        dt = sync_max(dt * 1e3) * 1e-3
        if rank == 0:
            print(json.dumps({
                "metric": "multi-mesh texture batch, meshes/s", "value": round(32 / dt, 3), "unit": "meshes/s",
                "n_gpus": world, "steps": 10, "warmup": 1, "ms_per_step": round(dt * 1e3 / (10 * len(mine)), 3),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 + W8A8 linears",
                "data": "synthetic",
                "config": {"workload": "32 meshes x 10 INT8 denoise steps, seeds 0..31 sharded round-robin, "
                                       "bf16 latents gathered on rank 0 (BASELINE configs[4])", "quant": args.quant},
                "missing": missing, "collected": len(results),
            }), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps (default: 400 sweep passes, 50 UNet forwards, 5 CPU reference passes)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense_sweep", choices=["dense_sweep", "sparse_sweep", "unet", "multimesh"])
    ap.add_argument("--quant", default="mixed", choices=["mixed", "dense", "sparse", "none"])
    ap.add_argument("--cpu-frac", type=float, default=None,
                    help="row fraction of each shape timed on the CPU (default: all rows, fewer when "
                         "the requested number of reference passes would take more than ~2 minutes)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.steps is None:
        args.steps = 5 if args.impl == "reference" else (50 if args.workload in ("unet", "multimesh") else 400)
    if args.cpu_frac is None:
        # One pass over all rows takes ~0.6 s on the host cores of the GPU box.
        args.cpu_frac = 1.0
        if args.impl == "reference":
            args.cpu_frac = min(1.0, 120.0 / (0.6 * (args.steps + args.warmup)))
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("unet", "multimesh"):
        run_unet(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
