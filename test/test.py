#!/usr/bin/env python
"""Speed test: overlapped GEMM+collective vs its parts and vs the cuBLAS+NCCL baseline.

    python test/test.py --m 4096 --n 8192 --k 8192 --comm_op all_reduce
    torchrun --nproc-per-node 8 test/test.py --m 8192 --n 8192 --k 3584

Reports, as the reference's test does (test/test.py:325-371): the GEMM alone, the bare
collective, the non-overlapped baseline (cuBLAS GEMM then one NCCL call), the overlapped op and
the speedup baseline/overlap - here for both overlap mechanisms (fused in-kernel collective and
the counter-gated NCCL scheme) - plus the fraction of the roofline the fused op reaches.  K is
the per-rank K.  A tuned ``configs/m{M}n{N}k{K}_{gpu}.json`` is used when present, otherwise an
untuned default (analytic hint, Algo 1).
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tune"))

import torch  # noqa: E402

from _common import OverlapWorkload, dtype_of  # noqa: E402

from flashoverlap_b200 import tuner  # noqa: E402
from flashoverlap_b200.parallel import bootstrap  # noqa: E402
from flashoverlap_b200.parallel.launch import run_on_all_gpus  # noqa: E402
from flashoverlap_b200.utils import config, layout  # noqa: E402
from flashoverlap_b200.utils.timing import perf_ms  # noqa: E402

WARM_UP = 20
REP = 200


def worker(rank, world, args):
    dt = dtype_of(args.dtype)
    impl = bootstrap.make_overlap_impl(rank, world)
    impl.set_option("timeout_ms", args.timeout_ms)
    base = bootstrap.make_baseline_impl(rank, world)

    def checked(fn):
        """One call, then the device status: a protocol failure stops the test here instead of
        running into the bounded waits again on every timed iteration."""
        fn()
        torch.cuda.synchronize()
        impl.check_status()
        return fn

    # a tuned config counts only if it was searched for this world size and collective
    cfg = config.load_tuned(args.m, args.n, args.k, tp=world, comm_op=args.comm_op, directory=args.path) or \
        config.default_solution(args.m, args.n, args.algo)
    algo = cfg["Algo"]
    sm, margin = impl.get_option("sm_count"), impl.get_option("sm_margin")
    res = {"M": args.m, "N": args.n, "K": args.k, "tp": world, "comm_op": args.comm_op, "Algo": algo}

    wl = OverlapWorkload(impl, rank, world, args.m, args.n, args.k, algo, args.comm_op, dt, mode="fused",
                         cseg=cfg["cSeg"] if cfg.get("mode", "fused") == "fused" else None, hint=cfg["hint"])
    f = args.flush
    res["gemm_ms"] = perf_ms(lambda: impl.cutlass_gemm(wl.A, wl.B, wl.C, algo), WARM_UP, args.reps, f)
    res["cublas_gemm_ms"] = perf_ms(lambda: base.cublas_gemm(wl.A, wl.B, wl.C), WARM_UP, args.reps, f)
    full = torch.empty(args.m, args.n, device=wl.dev, dtype=dt)
    comm = (lambda: impl.nccl_allreduce(full)) if args.comm_op == "all_reduce" else (lambda: impl.nccl_reducescatter(full))
    res["comm_ms"] = perf_ms(comm, WARM_UP, args.reps, f)
    if args.comm_op == "all_reduce":
        res["baseline_ms"] = perf_ms(lambda: base.gemm_allreduce(wl.A, wl.B, full), WARM_UP, args.reps, f)
    else:
        res["baseline_ms"] = perf_ms(lambda: base.gemm_reducescatter(wl.A, wl.B, full, wl.D), WARM_UP, args.reps, f)
    res["nonoverlap_ms"] = perf_ms(wl.run_nonoverlap, WARM_UP, args.reps, f)
    wl.set_cseg([1] * wl.tiles if "cSeg" not in cfg or cfg.get("mode") == "gated" else cfg["cSeg"])
    res["fused_ms"] = perf_ms(checked(wl.run), WARM_UP, args.reps, f)
    if world > 1 and args.pull:
        # pull protocol: partials stay on the producing GPU; owners fetch them with peer loads,
        # then (staging with a multicast mapping) with one switch-side reduction per vector
        from flashoverlap_b200.parallel import symm
        impl.set_option("stage_local", 1)
        res["fused_pull_peer_ms"] = perf_ms(checked(wl.run), WARM_UP, args.reps, f)
        _, switch = symm.alloc_stage(impl, args.m, args.n, dt)
        if switch:
            for direct in (0, 1):
                impl.set_option("pull_direct", direct)
                res["fused_pull_switch_direct_ms" if direct else "fused_pull_switch_ms"] = \
                    perf_ms(checked(wl.run), WARM_UP, args.reps, f)
            impl.set_option("pull_direct", -1)
        impl.set_option("stage_local", 0)
    if world > 1 and args.epi4:
        impl.set_option("epi_bufs", 4)
        res["fused_epi4_ms"] = perf_ms(checked(wl.run), WARM_UP, args.reps, f)
        impl.set_option("epi_bufs", 2)
    if world > 1:
        wl.mode = "gated"
        wave = sm - margin
        nw = layout.div_up(wl.tiles, wave)
        cseg = cfg["cSeg"] if cfg.get("mode") == "gated" else \
            layout.cseg_from_wave_groups(wl.tiles, wave, [nw // 4 + (1 if i < nw % 4 else 0) for i in range(4)]
                                         if nw >= 4 else [1] * nw)
        wl.C = full
        wl.set_cseg(cseg)
        res["gated_ms"] = perf_ms(wl.run, WARM_UP, args.reps, f)
    impl.check_status()
    peaks = {"bf16_tflops": 1590.0}
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    roof = tuner.roofline_ms(args.m, args.n, args.k, world, args.comm_op, peaks["bf16_tflops"], 770.0)
    res["roofline_ms"] = roof
    res["roofline_frac"] = roof / res["fused_ms"]
    res["speedup_fused"] = res["baseline_ms"] / res["fused_ms"]
    if "gated_ms" in res:
        res["speedup_gated"] = res["baseline_ms"] / res["gated_ms"]
    if rank == 0:
        print(f"m={args.m} n={args.n} k={args.k} tp={world} {args.comm_op} Algo={algo}")
        print(f"{'gemm (ours)':>24} {res['gemm_ms']:.4f} ms   {'gemm (cuBLAS)':>16} {res['cublas_gemm_ms']:.4f} ms")
        print(f"{'comm (NCCL)':>24} {res['comm_ms']:.4f} ms")
        print(f"{'baseline cuBLAS+NCCL':>24} {res['baseline_ms']:.4f} ms")
        print(f"{'our GEMM + NCCL':>24} {res['nonoverlap_ms']:.4f} ms")
        if "gated_ms" in res:
            print(f"{'overlap (gated NCCL)':>24} {res['gated_ms']:.4f} ms   speedup {res['speedup_gated']:.3f}")
        print(f"{'overlap (fused)':>24} {res['fused_ms']:.4f} ms   speedup {res['speedup_fused']:.3f}   "
              f"roofline {res['roofline_ms']:.4f} ms ({100 * res['roofline_frac']:.1f}% of measured peaks)")
        for key, label in (("fused_pull_peer_ms", "fused, pull (peer loads)"), ("fused_pull_switch_ms", "fused, pull (switch sum)"),
                           ("fused_pull_switch_direct_ms", "pull (switch), direct st"),
                           ("fused_epi4_ms", "fused, 4 chunk buffers")):
            if key in res:
                print(f"{label:>24} {res[key]:.4f} ms   speedup {res['baseline_ms'] / res[key]:.3f}")
        print(json.dumps({k: (round(v, 5) if isinstance(v, float) else v) for k, v in res.items()}))
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--comm_op", default="all_reduce", choices=["all_reduce", "reduce_scatter"])
    ap.add_argument("--algo", type=int, default=1)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--path", default=None)
    ap.add_argument("--reps", type=int, default=REP)
    ap.add_argument("--flush", action="store_true", help="flush L2 between timed iterations")
    ap.add_argument("--timeout_ms", type=int, default=5000, help="bound of the kernels' cross-GPU waits")
    ap.add_argument("--epi4", action="store_true",
                    help="also time the fused kernel built with four epilogue chunk buffers (option epi_bufs)")
    ap.add_argument("--pull", action="store_true",
                    help="also time the pull protocol of the fused kernel (option stage_local), with peer loads "
                         "and with the NVSwitch reduction")
    args = ap.parse_args()
    run_on_all_gpus(worker, args)


if __name__ == "__main__":
    main()
