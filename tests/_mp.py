"""Helpers for tests that run several ranks as child processes on this machine."""
import os
import socket
import tempfile
import time
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _leave_together(rank, world, result_dir, ok, limit_s=20.0):
    """A rank must not unmap its device memory while a peer's kernel may still address it (peer
    or multicast mappings): before leaving, every rank drops a marker and waits - bounded - until
    all ranks have dropped theirs.  Kernels' own waits are bounded by a few seconds, so after the
    limit nothing of the other ranks is in flight either way."""
    open(os.path.join(result_dir, f"r{rank}.{'left' if ok else 'failed'}"), "w").close()
    t0 = time.time()
    while time.time() - t0 < limit_s:
        if all(os.path.exists(os.path.join(result_dir, f"r{r}.left")) or
               os.path.exists(os.path.join(result_dir, f"r{r}.failed")) for r in range(world)):
            return
        time.sleep(0.05)


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
        if backend == "nccl":
            torch.cuda.synchronize()
        _leave_together(rank, world, result_dir, True)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(result_dir, f"r{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        _leave_together(rank, world, result_dir, False)
        raise


def run_ranks(fn, world: int, backend: str = "gloo", args=(), timeout_s: int = 60):
    """Runs fn(rank, world, *args) in `world` processes; returns the per-rank results.

    The rendezvous port is picked by binding to port 0 and closing the socket, so another process
    (or a lingering socket of the previous test) can take it before rank 0 listens on it; a run
    that fails with "address already in use" is repeated on a fresh port, twice at most."""
    for attempt in range(3):
        with tempfile.TemporaryDirectory() as d:
            try:
                mp.spawn(_entry, args=(world, backend, free_port(), fn, args, d, timeout_s), nprocs=world, join=True)
            except Exception as ex:
                errs = []
                for r in range(world):
                    p = os.path.join(d, f"r{r}.err")
                    if os.path.exists(p):
                        errs.append(f"--- rank {r} ---\n" + open(p).read())
                text = "\n".join(errs) + f"\n{ex}"
                if attempt < 2 and ("EADDRINUSE" in text or "address already in use" in text):
                    time.sleep(1.0)
                    continue
                raise AssertionError("rank failure:\n" + text) from ex
            return [torch.load(os.path.join(d, f"r{r}.pt"), weights_only=False) for r in range(world)]
