#!/usr/bin/env python
"""Shape sweep: fused GEMM+collective vs cuBLAS+NCCL, roofline fraction, and the tuner's predicted
vs exhaustive-best wave grouping.

    torchrun --nproc-per-node 8 test/sweep.py                 # tp = number of ranks
    python test/sweep.py --quick --out sweep_tp2.jsonl        # spawns one process per GPU

Shapes: M in {1024,2048,4096,8192,16384} x N in {4096,8192} x K_total in {8192,14336,28672} split
over the ranks, bf16 ~N(0,0.02), for all_reduce and reduce_scatter.  One JSON line per case:
latencies (device events, max over ranks), speedup over cuBLAS+NCCL, achieved fraction of the
roofline max(GEMM at measured tensor peak, bytes over NVLink at 770 GB/s), and - with
``--groupings`` - the gated mechanism's predicted and exhaustive-best cSeg.
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


def worker(rank, world, args):
    import torch.distributed as dist
    dt = dtype_of("bf16")
    base = bootstrap.make_baseline_impl(rank, world)
    peaks = {"bf16_tflops": 1590.0}
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    Ms = [1024, 4096, 16384] if args.quick else [1024, 2048, 4096, 8192, 16384]
    Ns = [8192] if args.quick else [4096, 8192]
    Ks = [8192, 28672] if args.quick else [8192, 14336, 28672]
    out = []
    for comm_op in ("all_reduce", "reduce_scatter"):
        for M in Ms:
            for N in Ns:
                for Kt in Ks:
                    K = Kt // world
                    # a fresh runtime object per case: its symmetric memory is released with it
                    impl = bootstrap.make_overlap_impl(rank, world)
                    impl.set_option("timeout_ms", 20000)
                    if getattr(args, "pull", False) and world > 1:
                        # pull protocol: partials staged locally, summed by the switch when the
                        # staging buffer gets a multicast mapping
                        from flashoverlap_b200.parallel import symm
                        symm.alloc_stage(impl, M, N, dt)
                        impl.set_option("stage_local", 1)
                    sm, margin = impl.get_option("sm_count"), impl.get_option("sm_margin")
                    best = None
                    for algo in ((19, 17, 1) if M % 512 == 0 else ((1, 17) if M % 256 == 0 else (0, 16))):
                        wl = OverlapWorkload(impl, rank, world, M, N, K, algo, comm_op, dt, mode="fused")
                        wl.set_cseg([1] * wl.tiles)
                        t = perf_ms(wl.run, args.warmup, args.reps, args.flush)
                        if best is None or t < best[0]:
                            best = (t, algo)
                        del wl
                    fused_ms, algo = best
                    wl = OverlapWorkload(impl, rank, world, M, N, K, algo, comm_op, dt, mode="fused")
                    full = torch.empty(M, N, device=wl.dev, dtype=dt)
                    if comm_op == "all_reduce":
                        base_ms = perf_ms(lambda: base.gemm_allreduce(wl.A, wl.B, full), args.warmup, args.reps, args.flush)
                    else:
                        base_ms = perf_ms(lambda: base.gemm_reducescatter(wl.A, wl.B, full, wl.D), args.warmup, args.reps, args.flush)
                    gemm_ms = perf_ms(lambda: impl.cutlass_gemm(wl.A, wl.B, full, algo), args.warmup, args.reps, args.flush)
                    roof = tuner.roofline_ms(M, N, K, world, comm_op, peaks["bf16_tflops"], 770.0)
                    rec = {"comm_op": comm_op, "M": M, "N": N, "K_total": Kt, "tp": world, "Algo": algo,
                           "protocol": "pull" if (getattr(args, "pull", False) and world > 1) else "push",
                           "fused_ms": round(fused_ms, 5), "cublas_nccl_ms": round(base_ms, 5), "gemm_ms": round(gemm_ms, 5),
                           "speedup": round(base_ms / fused_ms, 4), "roofline_ms": round(roof, 5),
                           "roofline_frac": round(roof / fused_ms, 4)}
                    if args.groupings and world > 1:
                        # fused mechanism: wave groups only coarsen the arrival counters; the search
                        # space is the same compositions plus one counter per tile
                        grid = min(sm * config.algo_params(algo)["mt"], wl.tiles)
                        f_cands = tuner.candidate_groupings(wl.tiles, grid, max_waves_per_unit=4) + [[1] * wl.tiles]

                        def measure_fused(cseg):
                            wl.set_cseg(cseg)
                            return perf_ms(wl.run, args.warmup, args.reps, args.flush)

                        cs_e, t_e, _ = tuner.exhaustive_search(f_cands, measure_fused)
                        rec.update(fused_best_groups=len(cs_e), fused_best_ms=round(t_e, 5))
                        f_curve = config.bandwidth_path(comm_op, world, args.path).parent / f"bandwidth_fused_{comm_op}_tp{world}.pt"
                        if os.path.exists(f_curve):
                            prob = tuner.Problem(M, N, wl.BM, wl.BN, gemm_ms, sm, world, comm_op, grid=grid)
                            cs_p, t_p = tuner.predictive_search(prob, torch.load(f_curve), "fused", f_cands, grid)
                            t_pm = measure_fused(cs_p)
                            rec.update(fused_predicted_groups=len(cs_p), fused_predicted_model_ms=round(t_p, 5),
                                       fused_predicted_measured_ms=round(t_pm, 5),
                                       fused_pick_within=round(t_pm / t_e, 4), fused_model_error=round(t_p / t_pm - 1.0, 4))
                        curve_path = config.bandwidth_path(comm_op, world, args.path)
                        wave = sm - margin
                        wl.mode = "gated"
                        wl.C = full
                        cands = tuner.candidate_groupings(wl.tiles, wave, max_waves_per_unit=5)

                        def measure(cseg):
                            wl.set_cseg(cseg)
                            return perf_ms(wl.run, 3, max(5, args.reps // 4))

                        wl.mode = "gated"
                        cs_e, t_e, _ = tuner.exhaustive_search(cands, measure)
                        rec.update(gated_best_cseg=cs_e, gated_best_ms=round(t_e, 5))
                        if os.path.exists(curve_path):
                            prob = tuner.Problem(M, N, wl.BM, wl.BN, gemm_ms, sm, world, comm_op, sm_margin=margin)
                            cs_p, t_p = tuner.predictive_search(prob, torch.load(curve_path), "gated", cands, wave)
                            t_pm = measure(cs_p)
                            rec.update(gated_predicted_cseg=cs_p, gated_predicted_model_ms=round(t_p, 5),
                                       gated_predicted_measured_ms=round(t_pm, 5), gated_pick_within=round(t_pm / t_e, 4),
                                       gated_model_error=round(t_p / t_pm - 1.0, 4))
                    impl.check_status()
                    torch.cuda.synchronize()
                    if world > 1:
                        dist.barrier()          # nobody frees memory a peer may still address
                    del wl, full, impl
                    out.append(rec)
                    if rank == 0:
                        print(json.dumps(rec), flush=True)
                        if args.out:
                            with open(args.out, "a") as f:
                                f.write(json.dumps(rec) + "\n")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--groupings", action="store_true", help="also search the gated mechanism's wave groupings")
    ap.add_argument("--flush", action="store_true")
    ap.add_argument("--pull", action="store_true", help="fused kernels use the pull protocol (in-switch reduction)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--path", default=None)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    run_on_all_gpus(worker, args)


if __name__ == "__main__":
    main()
