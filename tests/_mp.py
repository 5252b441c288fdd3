"""Helpers for tests that run several ranks as child processes on this machine."""
import os
import socket
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, backend, port, fn, args, result_dir, timeout_s):
    import datetime
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s))
        out = fn(rank, world, *args)
        torch.save(out, os.path.join(result_dir, f"r{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(result_dir, f"r{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise


def run_ranks(fn, world: int, backend: str = "gloo", args=(), timeout_s: int = 60):
    """Runs fn(rank, world, *args) in `world` processes; returns the per-rank results."""
    with tempfile.TemporaryDirectory() as d:
        try:
            mp.spawn(_entry, args=(world, backend, free_port(), fn, args, d, timeout_s), nprocs=world, join=True)
        except Exception as ex:
            errs = []
            for r in range(world):
                p = os.path.join(d, f"r{r}.err")
                if os.path.exists(p):
                    errs.append(f"--- rank {r} ---\n" + open(p).read())
            raise AssertionError("rank failure:\n" + "\n".join(errs) + f"\n{ex}") from ex
        return [torch.load(os.path.join(d, f"r{r}.pt"), weights_only=False) for r in range(world)]
