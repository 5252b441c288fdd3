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


def _arm_watchdog() -> None:
    """FLASHOVERLAP_HANG_DUMP=<seconds>: every rank dumps its Python stacks to stderr if it is
    still running after that long, and again at the same interval - enough to see which
    collective or synchronisation a stuck rank is sitting in."""
    secs = float(os.environ.get("FLASHOVERLAP_HANG_DUMP", "0") or 0)
    if secs > 0:
        import faulthandler
        import sys
        faulthandler.dump_traceback_later(secs, repeat=True, file=sys.stderr)


def _child(rank: int, world: int, port: int, fn: Callable, args: tuple, out_path: str, backend: str) -> None:
    _arm_watchdog()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank),
                      WORLD_SIZE=str(world))
    if backend == "nccl":
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    else:
        dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        res = fn(rank, world, *args)
    except BaseException:
        # The peers may be blocked in a collective that this rank will never join, and a clean
        # process-group shutdown would wait for them: report and leave at once, the parent then
        # terminates the other ranks.
        import time
        import traceback
        traceback.print_exc()
        # Peers' kernels may still address this rank's memory (peer or multicast mappings);
        # their device waits are bounded, so give them a moment to run out before the mappings go.
        try:
            torch.cuda.synchronize()
        except Exception:
            pass
        time.sleep(float(os.environ.get("FLASHOVERLAP_EXIT_GRACE_S", "3")))
        os._exit(1)
    if rank == 0:
        torch.save(res, out_path)
    dist.barrier()
    dist.destroy_process_group()


def run_on_all_gpus(fn: Callable[..., Any], *args, nprocs: Optional[int] = None, backend: str = "nccl") -> Any:
    """``backend="gloo"`` with an explicit ``nprocs`` runs the same launcher on CPU ranks (tests)."""
    if backend != "nccl":
        with tempfile.TemporaryDirectory() as d:
            out = os.path.join(d, "rank0.pt")
            mp.spawn(_child, args=(nprocs, _free_port(), fn, args, out, backend), nprocs=nprocs, join=True)
            return torch.load(out, weights_only=False) if os.path.exists(out) else None
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        from .bootstrap import init_distributed
        _arm_watchdog()
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
        mp.spawn(_child, args=(world, _free_port(), fn, args, out, backend), nprocs=world, join=True)
        return torch.load(out, weights_only=False) if os.path.exists(out) else None
