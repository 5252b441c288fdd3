#!/usr/bin/env python
"""GEMM + ReduceScatter + RMSNorm: overlapped pipeline vs the plain PyTorch / NCCL pipeline.

    python example/correctness_rs.py --m 4096 --n 4096 --k 8192

Mirrors the reference's script (example/correctness_rs.py:21-71): the overlapped reduce-scatter
hands rank p the rows ``i % world == p``, so the reference pipeline is fed the rows regrouped by
``reorder_rows_by_world_size`` and both sides end with the same local shard.  K is per rank.
"""
import argparse

import _common  # noqa: F401
import torch
import torch.nn as nn

from flashoverlap_b200.models import OverlapRowParallelLayer, ReorderRMSNorm, RMSNorm, RowParallelLayer
from flashoverlap_b200.parallel import bootstrap
from flashoverlap_b200.parallel.launch import run_on_all_gpus
from flashoverlap_b200.utils import config
from flashoverlap_b200.utils.layout import reorder_rows_by_world_size


def worker(rank, world, args):
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    M, N, K = args.m, args.n, args.k
    cfg = config.load_tuned(M, N, K, tp=world, comm_op="reduce_scatter", directory=args.path) or \
        config.default_solution(M, N, args.algo)
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(200 + rank)
    A0 = (torch.randn(M, K, device=dev, generator=g) * 0.5).to(dt)
    A1 = reorder_rows_by_world_size(A0, world)
    B = (torch.randn(N, K, device=dev, generator=g) * 0.5).to(dt)
    gw = torch.Generator(device=dev).manual_seed(7)
    W = (1 + 0.02 * torch.randn(N, device=dev, generator=gw)).to(dt)

    norm = RMSNorm(N, eps=1e-5, dtype=dt)
    norm.weight = nn.Parameter(W)
    rnorm = ReorderRMSNorm(N, M // world, cfg["BM"] // world, cfg["BN"], cfg["hint"], eps=1e-5, dtype=dt)
    rnorm.weight = nn.Parameter(W)
    ref_layer = RowParallelLayer(K, N, "reduce_scatter", None, dtype=dt)
    ref_layer.weight = nn.Parameter(B)
    nccl_id = bootstrap.share_nccl_id(rank, world)
    ov_layer = OverlapRowParallelLayer(rank, world, K, N, M, cfg, "reduce_scatter", nccl_id, dtype=dt, mode=args.mode)
    ov_layer.weight = nn.Parameter(B)

    torch.cuda.synchronize()
    with torch.no_grad():
        y1 = norm(ref_layer(A1))
        y2 = rnorm(ov_layer(A0))
    torch.cuda.synchronize()
    ov_layer.overlap_class.check_status()
    diff = (y1.float() - y2.float()).abs()
    ok = torch.allclose(y1.float(), y2.float(), atol=5e-2, rtol=5e-2)
    if rank == 0:
        i = torch.unravel_index(diff.argmax(), diff.shape)
        print(f"max abs diff {diff.max().item():.5f} at {tuple(int(x) for x in i)}: {y1[i].item():.4f} vs {y2[i].item():.4f}")
        print("[GEMM+ReduceScatter+RMSNorm] all close : ", ok)
    return ok


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--algo", type=int, default=1)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--mode", default="fused", choices=["fused", "gated"])
    ap.add_argument("--path", default=None)
    args = ap.parse_args()
    ok = run_on_all_gpus(worker, args)
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
