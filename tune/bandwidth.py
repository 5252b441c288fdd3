#!/usr/bin/env python
"""Bandwidth curves of the collectives, for the predictive search.

    python tune/bandwidth.py --comm_op all_reduce            # spawns one process per GPU
    torchrun --nproc-per-node 8 tune/bandwidth.py --comm_op reduce_scatter

For 36 message sizes (2**20 .. 2**28.75 fp16/bf16 elements) two curves are measured and saved as
``[36, 2]`` tensors of (elements, GiB/ms of algorithmic bytes):

* ``configs/bandwidth_{op}_tp{ws}.pt``        - the NCCL collective (what the reference measures,
  tune/bandwidth.py:48-111), used for ``mode=gated``;
* ``configs/bandwidth_fused_{op}_tp{ws}.pt``  - the in-kernel collective of the fused GEMM: the
  fused kernel on a [rows, 8192] output with K = 64, so that the time is the NVLink push +
  reduce + write-back, not the math.

A plot is written next to them with the headless Agg backend (the reference calls
``plt.show()``, which needs a display).
"""
import argparse

from _common import config, dtype_of, torch


from flashoverlap_b200 import tuner
from flashoverlap_b200.parallel import bootstrap
from flashoverlap_b200.parallel.launch import run_on_all_gpus
from flashoverlap_b200.utils.timing import perf_ms


def worker(rank, world, comm_op, dtype, path, warmup, reps):
    dt = dtype_of(dtype)
    impl = bootstrap.make_overlap_impl(rank, world)
    sizes = tuner.bandwidth_sizes()
    nccl_ms, fused_ms = [], []
    N = 8192
    for n in sizes:
        x = torch.zeros(1024, n // 1024, device="cuda", dtype=dt)
        fn = (lambda: impl.nccl_allreduce(x)) if comm_op == "all_reduce" else (lambda: impl.nccl_reducescatter(x))
        nccl_ms.append(perf_ms(fn, warmup, reps))
        rows = max(256, (n // N) // 256 * 256)
        A = torch.zeros(rows, 64, device="cuda", dtype=dt)
        B = torch.zeros(N, 64, device="cuda", dtype=dt)
        if comm_op == "all_reduce":
            C = impl.symm_empty([rows, N], dtype)
            f2 = lambda: impl.gemm_allreduce_fused(A, B, C, 1)
        else:
            D = torch.empty(rows // world, N, device="cuda", dtype=dt)
            f2 = lambda: impl.gemm_reducescatter_fused(A, B, D, 1)
        t = perf_ms(f2, warmup, max(10, reps // 4)) if world > 1 else 0.0
        fused_ms.append(t * n / float(rows * N))           # scale to the nominal element count
        del x, A, B
    impl.check_status()
    if rank == 0:
        out = {"nccl": tuner.curve_from_timings(sizes, nccl_ms, comm_op, world),
               "fused": tuner.curve_from_timings(sizes, fused_ms, comm_op, world) if world > 1 else None}
        p = config.bandwidth_path(comm_op, world, path)
        p.parent.mkdir(parents=True, exist_ok=True)
        torch.save(out["nccl"], p)
        if out["fused"] is not None:
            torch.save(out["fused"], p.parent / f"bandwidth_fused_{comm_op}_tp{world}.pt")
        try:
            import matplotlib
            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
            plt.figure(figsize=(6, 4))
            plt.semilogx(out["nccl"][:, 0], out["nccl"][:, 1] * 2 ** 30 / 1e6, label="NCCL")
            if out["fused"] is not None:
                plt.semilogx(out["fused"][:, 0], out["fused"][:, 1] * 2 ** 30 / 1e6, label="in-kernel")
            plt.xlabel("elements"); plt.ylabel("GB/s (algorithmic)"); plt.legend(); plt.tight_layout()
            plt.savefig(p.parent / f"bandwidth_{comm_op}_tp{world}.png")
        except Exception as ex:   # plotting is optional
            print("plot skipped:", ex)
        for n, a, b in zip(sizes, nccl_ms, fused_ms):
            print(f"{n:>10d} elems  nccl {a:.4f} ms  fused {b:.4f} ms")
        return out
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--comm_op", default="all_reduce", choices=["all_reduce", "reduce_scatter"])
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--path", default=None)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--reps", type=int, default=200)
    args = ap.parse_args()
    run_on_all_gpus(worker, args.comm_op, args.dtype, args.path, args.warmup, args.reps)


if __name__ == "__main__":
    main()
