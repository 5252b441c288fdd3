#!/usr/bin/env python
"""Stage 1 of tuning: time every Algo of the tcgen05 GEMM on one GPU and keep the 10 fastest.

    python tune/profile_config.py --m 4096 --n 8192 --k 8192

Writes ``configs/m{M}n{N}k{K}_{gpu}.json`` with lists ``BM, BN, dur, Algo`` and refreshes
``configs/AlgoDict.pt`` (reference: tune/profile_config.py:57-93; it walks 102 CUTLASS
instantiations, we walk the Algo table of one hand-written kernel family).  K is the per-rank K.
"""
import argparse
import heapq

from _common import REP, WARM_UP, config, dtype_of, make_operands, torch

from flashoverlap_b200 import ops
from flashoverlap_b200.utils.timing import perf_ms


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--path", default=None, help="config directory (default: <repo>/configs)")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    dt = dtype_of(args.dtype)
    impl = ops.OverlapImpl()
    impl.nccl_init(0, 1, [0] * 16)
    impl.cutlass_init()
    A, B = make_operands(args.m, args.n, args.k, dt, "cuda")
    C = torch.empty(args.m, args.n, device="cuda", dtype=dt)
    timed = []
    for algo in range(config.NUM_ALGOS):
        p = config.algo_params(algo)
        if args.n % p["BN"] or args.m % (p["BM"] * p["rows_per_unit"]):
            continue
        ms = perf_ms(lambda: impl.cutlass_gemm(A, B, C, algo), WARM_UP, REP, reduce_max=False)
        timed.append((ms, algo))
        print(f"Algo {algo:2d} {config.algo_tuple(algo)}: {ms:.4f} ms "
              f"({2 * args.m * args.n * args.k / ms / 1e9:.0f} TFLOP/s)")
    best = heapq.nsmallest(10, timed)
    path = config.config_path(args.m, args.n, args.k, directory=args.path)
    config.save_stage1(path, [config.algo_params(a)["BM"] for _, a in best],
                       [config.algo_params(a)["BN"] for _, a in best], [t for t, _ in best], [a for _, a in best])
    config.save_algo_dict(path.parent / "AlgoDict.pt")
    impl.check_status()
    print(f"wrote {path}")


if __name__ == "__main__":
    main()
