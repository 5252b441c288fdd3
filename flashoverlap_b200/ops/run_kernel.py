"""Run one kernel of the library on one GPU a few times and print its device time.

    python -m flashoverlap_b200.ops.run_kernel --kernel gemm --m 8192 --n 8192 --k 8192 --algo 1
    python -m flashoverlap_b200.ops.run_kernel --kernel reorder_rmsnorm --m 16384 --n 8192
    python -m flashoverlap_b200.ops.run_kernel --kernel fused_ar --ranks 2 --m 4096 --n 4096 --k 2048 --algo 0

Meant for profilers and quick checks: few launches, fixed shapes, nothing else on the stream.
Kernels: ``gemm`` (tcgen05 GEMM, natural layout), ``gemm_reordered`` (tile-contiguous layout),
``cublas`` (library GEMM for comparison), ``rmsnorm``, ``reorder_rmsnorm``, ``reorder``,
``fused_ar`` / ``fused_rs`` (all ranks of the fused GEMM+collective emulated on this GPU in one
cooperative launch).
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import ops
from ..utils import config, layout


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True,
                    choices=["gemm", "gemm_reordered", "cublas", "rmsnorm", "reorder_rmsnorm", "reorder",
                             "fused_ar", "fused_rs"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--algo", type=int, default=1)
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", choices=["bf16", "fp16"], default="bf16")
    ap.add_argument("--trace", default=None, metavar="FILE.json",
                    help="fused kernels: record the per-tile timeline of one extra call, print its summary and "
                         "write a Chrome trace of rank 0")
    ap.add_argument("--epi-bufs", type=int, default=2, choices=[2, 4],
                    help="fused kernels: epilogue chunk buffers (4 = build with one operand stage fewer)")
    ap.add_argument("--stage-local", action="store_true",
                    help="fused kernels: pull protocol (partials staged locally, owners fetch them)")
    a = ap.parse_args()

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float16
    torch.manual_seed(0)
    M, N, K = a.m, a.n, a.k
    p = config.algo_params(a.algo)
    BM, BN = p["BM"], p["BN"]
    bytes_moved, flops = 0, 0

    if a.kernel in ("gemm", "gemm_reordered", "cublas"):
        A = (torch.randn(M, K, device=dev) * 0.02).to(dt)
        B = (torch.randn(N, K, device=dev) * 0.02).to(dt)
        C = torch.empty(M, N, device=dev, dtype=dt)
        flops = 2.0 * M * N * K
        if a.kernel == "cublas":
            fn = lambda: torch.matmul(A, B.t(), out=C)
        else:
            impl = ops.OverlapImpl()
            impl.nccl_init(0, 1, [0] * 16)
            impl.cutlass_init()
            if a.kernel == "gemm":
                fn = lambda: impl.cutlass_gemm(A, B, C, a.algo)
            else:
                cfg = config.default_solution(M, N, a.algo)
                RA = layout.reorder_indices((M // BM) * (N // BN), cfg["hint"], device=dev)
                mm = torch.zeros(1, N // BN, device=dev, dtype=torch.int32)
                e = torch.empty(0, dtype=torch.int32)
                fn = lambda: impl.gemm_allreduce_overlap(A, B, C, mm, RA, 1, e, e.to(dev), a.algo, False)
    elif a.kernel in ("rmsnorm", "reorder_rmsnorm", "reorder"):
        x = torch.randn(M, N, device=dev).to(dt)
        w = torch.ones(N, device=dev, dtype=dt)
        y = torch.empty_like(x)
        RA = torch.randperm((M // BM) * (N // BN), device=dev, dtype=torch.int32)
        bytes_moved = 2 * M * N * 2
        if a.kernel == "rmsnorm":
            fn = lambda: ops.rmsnorm(x, w, 1e-5, out=y)
        elif a.kernel == "reorder_rmsnorm":
            fn = lambda: ops.reorder_rmsnorm(x, M, N, w, BM, BN, RA, 1e-5, out=y)
        else:
            fn = lambda: ops.reorder(x, BM, BN, RA, out=y)
    else:
        ws = a.ranks
        A = [(torch.randn(M, K, device=dev) * 0.02).to(dt) for _ in range(ws)]
        B = [(torch.randn(N, K, device=dev) * 0.02).to(dt) for _ in range(ws)]
        rows = M if a.kernel == "fused_ar" else M // ws
        out = [torch.empty(rows, N, device=dev, dtype=dt) for _ in range(ws)]
        op = "all_reduce" if a.kernel == "fused_ar" else "reduce_scatter"
        flops = 2.0 * M * N * K * ws
        fn = lambda: ops.fused_loopback(op, A, B, out, algo=a.algo, natural_out=True, stage_local=a.stage_local,
                                        epi_bufs=a.epi_bufs)

    for _ in range(a.warmup):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(a.iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / a.iters
    res = {"kernel": a.kernel, "M": M, "N": N, "K": K, "algo": a.algo, "ms": round(ms, 5)}
    if flops:
        res["tflops"] = round(flops / ms / 1e9, 1)
    if bytes_moved:
        res["gbs"] = round(bytes_moved / ms / 1e6, 1)
    if a.trace and a.kernel in ("fused_ar", "fused_rs"):
        from ..utils import trace
        tiles = (M // BM) * (N // BN)
        buf = trace.new_buffer(tiles, a.ranks, dev)
        ops.fused_loopback(op, A, B, out, algo=a.algo, natural_out=True, stage_local=a.stage_local, trace=buf)  # default build
        res["timeline_us"] = {k: {kk: round(vv, 2) for kk, vv in v.items()} for k, v in trace.summarize(buf, tiles).items()}
        trace.to_chrome_trace(buf, tiles, a.trace)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
