#!/usr/bin/env python
"""Stage 1 of tuning from a list of candidate kernels in a CSV file.

    python tune/gen_config.py --m 4096 --n 8192 --k 8192 [--csv m4096n8192k8192.gemm.csv]

The reference feeds this step with the CUTLASS profiler's CSV (tune/gen_config.py:46-120): it
takes the 10 fastest rows, maps their tile parameters to an Algo index through ``AlgoDict.pt``
and re-times them under its wrapper.  There is no external profiler for a hand-written kernel
family, so the CSV here is any table with the columns ``cta_m, cta_n, cta_k, stages, raster,
cta_group`` (one candidate per row, optional ``runtime`` column used only for the initial sort);
rows that do not name an existing Algo are reported and skipped, or - with ``--add_missing`` -
registered as new kernels through ``tool/generate_instances.py`` (rebuild, then run again).  Without ``--csv`` every Algo is
a candidate.  Output is identical to ``profile_config.py``.
"""
import argparse
import csv
import heapq

from _common import REP, WARM_UP, config, dtype_of, make_operands, torch

from flashoverlap_b200 import ops
from flashoverlap_b200.utils.timing import perf_ms


def candidates_from_csv(path, add_missing=False):
    table = config.algo_dict()
    rows = []
    with open(path) as f:
        for row in csv.DictReader(f):
            rows.append(row)
    rows.sort(key=lambda r: float(r.get("runtime", 0) or 0))
    out = []
    for r in rows[:10]:
        bm, bn, bk = int(r["cta_m"]), int(r["cta_n"]), int(r["cta_k"])
        grp = int(r.get("cta_group", 1) or 1)
        acc_stages = 1 if bm == 256 else 2     # 256 rows per CTA: two halves, accumulators fill TMEM
        raster = int(r["raster"])
        key = (bm, bn, bk, 128 * grp, bn, 16, grp, acc_stages, 64, int(r["stages"]), raster, 1)
        if key in table:
            out.append(table[key])
        elif add_missing:
            # what the reference's gen_config does with an unknown row (tune/gen_config.py:46-67):
            # register the combination - here a new kernel plus one Algo per raster strip - and
            # ask for a rebuild; the row is skipped in this run
            gi = _generator()
            spec = gi.load_spec()
            try:
                idx = gi.add_kernel(spec, bn, int(r["stages"]), grp - 1, bm // 128)
                if raster not in spec["rasters"]:
                    gi.add_raster(spec, raster)
                gi.save_spec(spec)
                gi.emit(spec)
                print(f"registered kernel {idx} for {key}: rebuild the library "
                      f"(python -c 'import __graft_entry__ as g; g.build()') and run this step again")
            except ValueError as ex:
                print(f"cannot build a kernel for {key}: {ex}")
        else:
            print(f"no kernel for {key}: skipped (--add_missing registers it through tool/generate_instances.py)")
    return out


def _generator():
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tool", "generate_instances.py")
    spec = importlib.util.spec_from_file_location("generate_instances", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--csv", default=None)
    ap.add_argument("--add_missing", action="store_true",
                    help="register CSV rows that name no existing kernel as new kernels (then rebuild)")
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--path", default=None)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    dt = dtype_of(args.dtype)
    algos = candidates_from_csv(args.csv, args.add_missing) if args.csv else list(range(config.NUM_ALGOS))
    impl = ops.OverlapImpl()
    impl.nccl_init(0, 1, [0] * 16)
    impl.cutlass_init()
    A, B = make_operands(args.m, args.n, args.k, dt, "cuda")
    C = torch.empty(args.m, args.n, device="cuda", dtype=dt)
    timed = []
    for algo in algos:
        p = config.algo_params(algo)
        if args.n % p["BN"] or args.m % (p["BM"] * p["rows_per_unit"]):
            continue
        timed.append((perf_ms(lambda: impl.cutlass_gemm(A, B, C, algo), WARM_UP, REP, reduce_max=False), algo))
    best = heapq.nsmallest(10, timed)
    path = config.config_path(args.m, args.n, args.k, directory=args.path)
    config.save_stage1(path, [config.algo_params(a)["BM"] for _, a in best],
                       [config.algo_params(a)["BN"] for _, a in best], [t for t, _ in best], [a for _, a in best])
    config.save_algo_dict(path.parent / "AlgoDict.pt")
    print(f"wrote {path}")


if __name__ == "__main__":
    main()
