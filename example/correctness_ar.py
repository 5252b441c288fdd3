#!/usr/bin/env python
"""GEMM + AllReduce + RMSNorm: overlapped pipeline vs the plain PyTorch / NCCL pipeline.

    python example/correctness_ar.py --m 4096 --n 4096 --k 8192       # one process per visible GPU
    torchrun --nproc-per-node 2 example/correctness_ar.py

Same scenario as the reference's script (example/correctness_ar.py:21-57) with two changes: the
operands are random (the reference uses all-ones inputs, with which a wrong tile permutation
cannot be seen) and bf16 is the default dtype.  K is the per-rank K.
"""
import argparse

import _common  # noqa: F401
import torch
import torch.nn as nn

from flashoverlap_b200.models import OverlapRowParallelLayer, ReorderRMSNorm, RMSNorm, RowParallelLayer
from flashoverlap_b200.parallel import bootstrap
from flashoverlap_b200.parallel.launch import run_on_all_gpus
from flashoverlap_b200.utils import config


def worker(rank, world, args):
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    M, N, K = args.m, args.n, args.k
    cfg = config.load_tuned(M, N, K, tp=world, comm_op="all_reduce", directory=args.path) or \
        config.default_solution(M, N, args.algo)
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    A = (torch.randn(M, K, device=dev, generator=g) * 0.5).to(dt)
    B = (torch.randn(N, K, device=dev, generator=g) * 0.5).to(dt)
    gw = torch.Generator(device=dev).manual_seed(7)
    W = (1 + 0.02 * torch.randn(N, device=dev, generator=gw)).to(dt)

    norm = RMSNorm(N, eps=1e-5, dtype=dt)
    norm.weight = nn.Parameter(W)
    rnorm = ReorderRMSNorm(N, M, cfg["BM"], cfg["BN"], cfg["hint"], eps=1e-5, dtype=dt)
    rnorm.weight = nn.Parameter(W)
    ref_layer = RowParallelLayer(K, N, "all_reduce", None, dtype=dt)
    ref_layer.weight = nn.Parameter(B)
    nccl_id = bootstrap.share_nccl_id(rank, world)
    ov_layer = OverlapRowParallelLayer(rank, world, K, N, M, cfg, "all_reduce", nccl_id, dtype=dt, mode=args.mode)
    ov_layer.weight = nn.Parameter(B)

    torch.cuda.synchronize()
    with torch.no_grad():
        y1 = norm(ref_layer(A))
        y2 = rnorm(ov_layer(A))
    torch.cuda.synchronize()
    ov_layer.overlap_class.check_status()
    ok = torch.allclose(y1.float(), y2.float(), atol=1e-2, rtol=1e-2)
    if rank == 0:
        print(f"max abs diff {(y1.float() - y2.float()).abs().max().item():.5f}")
        print("[GEMM+AllReduce+RMSNorm] all close : ", ok)
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
