#!/usr/bin/env python
"""Llama-3-70B-shaped decoder layer forward under TP + sequence parallelism.

    torchrun --nproc-per-node 8 example/decoder_layer.py --batch 4 --seq 4096
    python example/decoder_layer.py --tiny        # small shapes, any number of GPUs

Runs the layer with the NCCL path (matmul, then ``reduce_scatter_tensor``) and with the fused
GEMM+ReduceScatter kernels for ``o_proj`` and ``down_proj``, checks that both give the same
output and prints the time of each.  Random-init bf16 weights ~N(0, 0.02); hidden 8192, FFN 28672
(SwiGLU), 64 query / 8 KV heads, head_dim 128.
"""
import argparse
import json

import _common  # noqa: F401
import torch
import torch.distributed as dist

from flashoverlap_b200.models import DecoderConfig, TPDecoderLayer
from flashoverlap_b200.parallel import bootstrap
from flashoverlap_b200.parallel.launch import run_on_all_gpus
from flashoverlap_b200.utils.timing import perf_ms


def worker(rank, world, args):
    cfg = DecoderConfig.tiny() if args.tiny else DecoderConfig.llama3_70b()
    if args.tiny and world > 2:
        cfg.n_kv_heads = 8
    batch, seq = (2, 256) if args.tiny else (args.batch, args.seq)
    T = batch * seq
    impl = bootstrap.make_overlap_impl(rank, world)
    impl.set_option("timeout_ms", 20000)
    g = torch.Generator(device="cpu").manual_seed(5)
    x_full = torch.randn(T, cfg.hidden, generator=g).to(torch.bfloat16).cuda()
    res, outs = {}, {}
    for mode in ("nccl", "fused"):
        layer = TPDecoderLayer(cfg, rank, world, batch, seq, impl=mode, overlap_impl=impl, algo=args.algo, seed=3)
        rows = layer.shard_rows().cuda()
        x_sp = x_full[rows].contiguous()
        with torch.no_grad():
            y = layer(x_sp)
            res[mode] = perf_ms(lambda: layer(x_sp), args.warmup, args.reps)
        full = torch.zeros(T, cfg.hidden, device="cuda", dtype=torch.float32)
        full[rows] = y.float()
        if world > 1:
            dist.all_reduce(full)
        outs[mode] = full
        del layer
    impl.check_status()
    err = (outs["nccl"] - outs["fused"]).abs().max().item()
    scale = outs["nccl"].abs().max().item()
    res.update(max_abs_diff=err, out_scale=scale, tokens=T, tp=world, speedup=res["nccl"] / res["fused"])
    if rank == 0:
        print(json.dumps({k: (round(v, 5) if isinstance(v, float) else v) for k, v in res.items()}))
    return err <= 0.03 * scale + 1e-2


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--algo", type=int, default=1)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--reps", type=int, default=10)
    args = ap.parse_args()
    ok = run_on_all_gpus(worker, args)
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
