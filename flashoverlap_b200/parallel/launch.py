"""Run a function on every GPU of the node, one process per GPU.

Two ways in, one way out: under ``torchrun`` (RANK / WORLD_SIZE in the environment) the calling
process IS a rank and the function runs in place; otherwise the ranks are spawned from here with
``torch.multiprocessing.spawn``, as the reference's scripts do (test/test.py:180-184,
tune/search.py:172-176).  Either way the function receives ``(rank, world, *args)`` with
``torch.distributed`` initialised (NCCL) and its CUDA device selected; rank 0's return value is
handed back to the caller.
"""
from __future__ import annotations

import os
import socket
import tempfile
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _child(rank: int, world: int, port: int, fn: Callable, args: tuple, out_path: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank),
                      WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        res = fn(rank, world, *args)
        if rank == 0:
            torch.save(res, out_path)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def run_on_all_gpus(fn: Callable[..., Any], *args, nprocs: Optional[int] = None) -> Any:
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        from .bootstrap import init_distributed
        rank, world, _ = init_distributed()
        res = fn(rank, world, *args)
        if world > 1:
            dist.barrier()
        return res
    world = nprocs or torch.cuda.device_count()
    if world <= 1:
        torch.cuda.set_device(0)
        return fn(0, 1, *args)
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "rank0.pt")
        mp.spawn(_child, args=(world, _free_port(), fn, args, out), nprocs=world, join=True)
        return torch.load(out, weights_only=False) if os.path.exists(out) else None
