"""Device-side timing used by the tuner, the speed test and the examples: CUDA events on the
launching stream around every iteration, mean per rank, maximum over ranks (the reference's
protocol, test/test.py:112-119, :186-190), plus an optional L2 flush between iterations."""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

_flush_buf = {}


def flush_l2() -> None:
    """Overwrites a 256 MB buffer (B200's L2 holds 126 MB)."""
    dev = torch.cuda.current_device()
    if dev not in _flush_buf:
        _flush_buf[dev] = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush_buf[dev].zero_()


def perf_ms(fn: Callable[[], None], warmup: int = 20, reps: int = 200, flush: bool = False,
            reduce_max: bool = True) -> float:
    for _ in range(warmup):
        fn()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    torch.cuda.synchronize()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    for s, e in ev:
        if flush:
            flush_l2()
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    ms = sum(s.elapsed_time(e) for s, e in ev) / reps
    if reduce_max and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms
