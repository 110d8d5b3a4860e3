"""Runs one kernel of the library a few times on one shape, for profiler captures.

    python hunyuan3d-tools_b200/profile_case.py {dense|sparse|quant|prune|fused} MxKxN [launches]

Allocates synthetic operands of the given shape on the current device (int8 A / B, scales,
bias, bf16 activations and output), calls the C-ABI entry point ``launches`` times (default 3)
and checks the status codes.  Nothing is timed here: the profiler does that.
"""
import importlib
import os
import sys

import torch


def main(argv):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    build = importlib.import_module("hunyuan3d-tools_b200.csrc.build")
    tc = build.load_tc_gemm()
    sp = build.load_sparse_tc()
    lib = tc._lib
    kind = argv[1]
    M, K, N = (int(v) for v in argv[2].split("x"))
    reps = int(argv[3]) if len(argv) > 3 else 3
    dev = "cuda"
    x = torch.randn(M, K, device=dev).bfloat16()
    q = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev)
    s = torch.rand(M, device=dev) * 0.01
    w = torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev)
    ws = torch.rand(N, device=dev).bfloat16()
    b = torch.rand(N, device=dev).bfloat16()
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    st = torch.cuda.current_stream().cuda_stream
    if kind == "sparse":
        comp, meta = sp.sparse_prune_and_pack(w)
    if kind == "prune":
        comp = torch.empty(N, K // 2, dtype=torch.int8, device=dev)
        ld = 4 * ((K + 127) // 128)
        meta = torch.empty(N, ld, dtype=torch.int32, device=dev)
    for _ in range(reps):
        if kind == "dense":
            r = lib.hy3d_gemm_w8a8_dense(q.data_ptr(), w.data_ptr(), s.data_ptr(), ws.data_ptr(), 1,
                                         b.data_ptr(), 1, out.data_ptr(), 1, M, N, K, 0, 0, 0, st)
        elif kind == "sparse":
            r = lib.hy3d_gemm_w8a8_sparse24(q.data_ptr(), s.data_ptr(), comp.data_ptr(), meta.data_ptr(),
                                            meta.shape[1], ws.data_ptr(), 1, b.data_ptr(), 1,
                                            out.data_ptr(), 1, M, N, K, 0, 0, st)
        elif kind == "quant":
            r = lib.hy3d_quantize_rows(x.data_ptr(), 1, M, K, K, q.data_ptr(), s.data_ptr(), st)
        elif kind == "prune":
            r = lib.hy3d_prune_pack_24(w.data_ptr(), N, K, comp.data_ptr(), None, meta.data_ptr(), ld, st)
        elif kind == "fused":
            r = lib.hy3d_linear_w8a8_dense_fused(x.data_ptr(), 1, K, None, w.data_ptr(), ws.data_ptr(), 1,
                                                 b.data_ptr(), 1, out.data_ptr(), 1, M, N, K, 0, 0, st)
        else:
            raise SystemExit(f"unknown kernel kind {kind!r}")
        if r != 0:
            raise SystemExit(f"status {r}")
    torch.cuda.synchronize()
    if tc.device_status() != 0:
        raise SystemExit("device status non-zero")
    print("ok")


if __name__ == "__main__":
    main(sys.argv)
