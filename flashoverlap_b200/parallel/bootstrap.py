"""Process bootstrap: one process per GPU, the NCCL unique id created on one rank and handed
to the others.  The reference creates the id in the parent of ``mp.spawn`` and passes it as an
argument (test/test.py:173-184); under ``torchrun`` there is no parent, so the id travels
through the ``torch.distributed`` store instead."""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def env_rank_world() -> Tuple[int, int, int]:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def init_distributed(backend: Optional[str] = None) -> Tuple[int, int, int]:
    """Initialises torch.distributed from the environment (no-op for a single process)."""
    rank, world, local = env_rank_world()
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return rank, world, local


def share_nccl_id(rank: int, world: int) -> List[int]:
    """Rank 0 generates a NCCL unique id; every rank returns the same 16 int64 values."""
    if world == 1:
        return [0] * 16
    from .._build import load
    load()   # registers torch.ops.flashoverlap_op
    payload = [torch.ops.flashoverlap_op.generate_nccl_id() if rank == 0 else None]
    dist.broadcast_object_list(payload, src=0)
    return list(payload[0])


def make_overlap_impl(rank: int, world: int, nccl_id: Optional[List[int]] = None):
    """OverlapImpl initialised the way the reference's callers do it
    (example/RowParallelLinear.py:44-47): nccl_init, cutlass_init, overlap_init."""
    from .._build import load
    load()
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.nccl_init(rank, world, nccl_id if nccl_id is not None else share_nccl_id(rank, world))
    impl.cutlass_init()
    impl.overlap_init()
    return impl


def make_baseline_impl(rank: int, world: int, nccl_id: Optional[List[int]] = None):
    from .._build import load
    load()
    impl = torch.classes.flashoverlap_class.BaselineImpl()
    impl.nccl_init(rank, world, nccl_id if nccl_id is not None else share_nccl_id(rank, world))
    impl.cublas_init()
    return impl
