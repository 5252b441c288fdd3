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
import time

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
    if args.pull and world > 1:
        # pull protocol of the fused kernels: staging with an NVSwitch multicast mapping, so the
        # owners sum the partial tiles with one in-switch reduction per vector
        from flashoverlap_b200.parallel import symm
        symm.alloc_stage(impl, T, cfg.hidden, torch.bfloat16)
        impl.set_option("stage_local", 1)
    modes = [("nccl", "nccl", False), ("fused", "fused", False)] + ([("fused_norm_tail", "fused", True)] if world > 1 else [])
    for name, mode, tail in modes:
        layer = TPDecoderLayer(cfg, rank, world, batch, seq, impl=mode, overlap_impl=impl, algo=args.algo, seed=3,
                               fuse_norm=tail)
        rows = layer.shard_rows().cuda()
        x_sp = x_full[rows].contiguous()
        with torch.no_grad():
            y = layer(x_sp)
            # every arm settles under about a second of its own load first: the board runs at its
            # power cap, and an arm timed right after another one's cool start reads faster
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            layer(x_sp)
            torch.cuda.synchronize()
            one = torch.tensor([max(time.perf_counter() - t0, 1e-4)], device="cuda")
            if world > 1:
                dist.all_reduce(one, op=dist.ReduceOp.MAX)
            settle = int(min(200, args.settle_s / one.item()))
            res[name] = perf_ms(lambda: layer(x_sp), max(args.warmup, settle), args.reps)
            if not tail:
                # the two row-parallel projections alone (GEMM + reduce-scatter), same operand shapes
                attn = torch.randn(T, layer.q_local * cfg.head_dim, device="cuda").to(torch.bfloat16) * 0.1
                act = torch.randn(T, layer.ffn_local, device="cuda").to(torch.bfloat16) * 0.1
                res[name + "_o_proj"] = perf_ms(lambda: layer._row_parallel(attn, layer.wo), args.warmup, args.reps)
                res[name + "_down_proj"] = perf_ms(lambda: layer._row_parallel(act, layer.wd), args.warmup, args.reps)
                del attn, act
        mode = name
        full = torch.zeros(T, cfg.hidden, device="cuda", dtype=torch.float32)
        full[rows] = y.float()
        if world > 1:
            dist.all_reduce(full)
        outs[mode] = full
        del layer
    impl.check_status()
    err = (outs["nccl"] - outs["fused"]).abs().max().item()
    scale = outs["nccl"].abs().max().item()
    if "fused_norm_tail" in outs:
        res["max_abs_diff_norm_tail"] = (outs["nccl"] - outs["fused_norm_tail"]).abs().max().item()
        err = max(err, res["max_abs_diff_norm_tail"])
    res.update(max_abs_diff=err, out_scale=scale, tokens=T, tp=world, speedup=res["nccl"] / res["fused"],
               protocol="pull" if (args.pull and world > 1) else "push",
               row_parallel_share_nccl=(res["nccl_o_proj"] + res["nccl_down_proj"]) / res["nccl"],
               row_parallel_share_fused=(res["fused_o_proj"] + res["fused_down_proj"]) / res["fused"])
    if rank == 0:
        print(json.dumps({k: (round(v, 5) if isinstance(v, float) else v) for k, v in res.items()}))
    return err <= 0.03 * scale + 1e-2


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--algo", type=int, default=1)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--pull", action="store_true", help="fused kernels use the pull protocol (in-switch reduction)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--settle_s", type=float, default=1.0, help="seconds of load before each arm is timed")
    args = ap.parse_args()
    ok = run_on_all_gpus(worker, args)
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
