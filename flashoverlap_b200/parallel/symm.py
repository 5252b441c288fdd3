"""Symmetric buffers for the fused collectives: AllReduce outputs and pull-protocol staging.

``alloc_allreduce_output`` returns a tensor that every rank can address.  When
``torch.distributed._symmetric_memory`` can provide it, the buffer also carries an NVSwitch
*multicast* mapping, and the kernel's reducers then broadcast each result vector with a single
``multimem.st`` (the switch replicates it to all GPUs) instead of one peer store per rank - which
halves the NVLink bytes an AllReduce puts on each GPU's links.  Otherwise the buffer comes from
the runtime's own IPC-based symmetric heap and results travel as peer-to-peer stores.  The
reference has no counterpart (its collectives are NCCL calls).
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch
import torch.distributed as dist

_DTYPE_NAMES = {torch.bfloat16: "bfloat16", torch.float16: "float16", torch.float32: "float32"}
_keepalive = []


def alloc_allreduce_output(impl, shape: Sequence[int], dtype=torch.bfloat16, group=None,
                           multicast: bool = True) -> Tuple[torch.Tensor, bool]:
    """Collective.  Returns (tensor, uses_multicast)."""
    return _alloc(impl, shape, dtype, group, multicast)


def alloc_stage(impl, M: int, N: int, dtype=torch.bfloat16, group=None,
                multicast: bool = True) -> Tuple[torch.Tensor, bool]:
    """Collective.  Staging buffer for the pull protocol of the fused kernels (option
    ``stage_local``): [M, N] 16-bit elements per rank, handed to the runtime with ``use_stage``.
    With a multicast mapping the owners' reducers fetch the sum of all ranks' partials with one
    ``multimem.ld_reduce`` per vector - the NVSwitch does the addition and only the result crosses
    the owner's links.  Returns (tensor, uses_multicast)."""
    t, mc = _alloc(impl, (M, N), dtype, group, multicast)
    if impl.get_option("world") > 1:
        impl.use_stage(t)
    return t, mc


def _alloc(impl, shape, dtype, group, multicast):
    world = impl.get_option("world")
    if world == 1:
        return torch.empty(*shape, dtype=dtype, device="cuda"), False
    ok, out, mc = 0, None, 0
    if multicast and dist.is_initialized() and dist.get_world_size(group) == world:
        try:
            import torch.distributed._symmetric_memory as symm_mem
            dev = torch.device("cuda", torch.cuda.current_device())
            t = symm_mem.empty(*shape, dtype=dtype, device=dev)
            hdl = symm_mem.rendezvous(t, group=group if group is not None else dist.group.WORLD)
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            if mc != 0 and len(ptrs) == world:
                out, ok = (t, hdl, ptrs), 1
        except Exception:
            ok = 0
        flag = torch.tensor([ok], device="cuda", dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)      # all ranks or none
        ok = int(flag.item())
    if ok:
        t, hdl, ptrs = out
        impl.register_symmetric(t, ptrs, mc)
        _keepalive.append((t, hdl))            # the mapping must outlive the runtime's use of it
        return t, True
    return impl.symm_empty(list(shape), _DTYPE_NAMES[dtype]), False
