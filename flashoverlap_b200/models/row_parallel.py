"""Row-parallel linear layers (reference: example/RowParallelLinear.py:8-82).

``RowParallelLayer`` is the unfused PyTorch reference: ``x @ W^T`` then ``dist.all_reduce`` or
``dist.reduce_scatter_tensor``.  ``OverlapRowParallelLayer`` owns an ``OverlapImpl`` and calls
the fused GEMM+collective kernels; constructor arguments follow the reference so its scripts
keep working, with optional extras.
"""
from __future__ import annotations


import torch
import torch.distributed as dist
import torch.nn as nn

from ..utils import layout


class RowParallelLayer(nn.Module):
    def __init__(self, in_features: int, out_features: int, comm_op: str, tp_group=None,
                 dtype=torch.bfloat16, device=None):
        super().__init__()
        if comm_op not in ("all_reduce", "reduce_scatter"):
            raise ValueError(f"comm_op must be 'all_reduce' or 'reduce_scatter', got {comm_op!r}")
        self.tp_group = tp_group
        self.comm_op = comm_op
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.weight = nn.Parameter(torch.randn(out_features, in_features, dtype=dtype, device=device) * 0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.matmul(x, self.weight.t())
        if not dist.is_initialized() or dist.get_world_size(self.tp_group) == 1:
            return out
        if self.comm_op == "all_reduce":
            dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.tp_group)
            return out
        ws = dist.get_world_size(self.tp_group)
        shard = torch.empty((x.size(0) // ws, self.weight.size(0)), dtype=out.dtype, device=out.device)
        dist.reduce_scatter_tensor(shard, out, group=self.tp_group)
        return shard


class OverlapRowParallelLayer(nn.Module):
    """``config`` is a tuned JSON dict (BM, BN, Algo, hint, cSeg).

    ``layout`` selects what ``forward`` returns:
      * ``"reordered"`` (default, reference behaviour): the tile-contiguous buffer, to be consumed
        by :class:`ReorderRMSNorm`;
      * ``"natural"``: row-major output written directly by the fused kernel (no reorder pass is
        needed at all, because the in-kernel collective does not require contiguous ranges).

    ``protocol`` (fused mode, several ranks): ``"push"`` - partial tiles are stored into the owning
    ranks' staging buffers - or ``"pull"`` - they stay in this rank's staging buffer, allocated
    here with an NVSwitch multicast mapping when torch can provide one, and the owners sum them
    with one in-switch reduction per vector (``multimem.ld_reduce``).
    """

    def __init__(self, rank: int, world_size: int, in_features: int, out_features: int, M: int,
                 config: dict, comm_op: str, nccl_id, dtype=torch.bfloat16, layout_mode: str = "reordered",
                 impl=None, mode: str = "fused", protocol: str = "push"):
        super().__init__()
        if comm_op not in ("all_reduce", "reduce_scatter"):
            raise ValueError(f"comm_op must be 'all_reduce' or 'reduce_scatter', got {comm_op!r}")
        from .._build import load
        load()
        self.weight = nn.Parameter(torch.randn(out_features, in_features, dtype=dtype, device="cuda") * 0.02)
        self.world_size = world_size
        self.comm_op = comm_op
        self.layout_mode = layout_mode
        self.M = M
        if impl is None:
            impl = torch.classes.flashoverlap_class.OverlapImpl()
            impl.nccl_init(rank, world_size, nccl_id)
            impl.cutlass_init()
            impl.overlap_init()
        self.overlap_class = impl
        impl.set_option("mode", 0 if mode == "fused" else 1)

        BM, BN = config["BM"], config["BN"]
        tm, tn = layout.div_up(M, BM), layout.div_up(out_features, BN)
        self.algo = config["Algo"]
        self.counter = torch.zeros((1, max(tn, len(config["cSeg"]))), dtype=torch.int32, device="cuda")
        self.reorder_array = layout.reorder_indices(tm * tn, config["hint"], device="cuda").reshape(tm, tn)
        self.cseg_cpu = torch.tensor(config["cSeg"], dtype=torch.int32)
        self.cseg_gpu = self.cseg_cpu.cuda()
        self.row_array = (layout.generate_row_mapping(M, out_features, BM, BN, config["cSeg"], world_size,
                                                      device="cuda")
                          if comm_op == "reduce_scatter" else torch.zeros(1, dtype=torch.int32, device="cuda"))
        # AllReduce results land in symmetric memory so that peers can write them directly.
        self._out = None
        if comm_op == "all_reduce" and world_size > 1 and mode == "fused":
            # symmetric memory, with an NVSwitch multicast mapping when torch can provide one
            from ..parallel import symm
            self._out, self.uses_multicast = symm.alloc_allreduce_output(impl, (M, out_features), dtype)
        self._tmp = None
        if protocol not in ("push", "pull"):
            raise ValueError(f"protocol must be 'push' or 'pull', got {protocol!r}")
        self.protocol = protocol if (world_size > 1 and mode == "fused") else "push"
        if self.protocol == "pull":
            from ..parallel import symm
            self._stage, self.stage_multicast = symm.alloc_stage(impl, M, out_features, dtype)
        if world_size > 1 and mode == "fused":
            impl.set_option("stage_local", 1 if self.protocol == "pull" else 0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        N = self.weight.size(0)
        if self.comm_op == "all_reduce":
            out = self._out if (self._out is not None and x.size(0) == self.M) else \
                torch.empty((x.size(0), N), dtype=x.dtype, device=x.device)
            if self.layout_mode == "natural":
                self.overlap_class.gemm_allreduce_fused(x, self.weight, out, self.algo)
            else:
                self.overlap_class.gemm_allreduce_overlap(
                    x, self.weight, out, self.counter, self.reorder_array, 1, self.cseg_cpu, self.cseg_gpu,
                    self.algo, False)
            return out
        out = torch.empty((x.size(0) // self.world_size, N), dtype=x.dtype, device=x.device)
        if self.layout_mode == "natural":
            self.overlap_class.gemm_reducescatter_fused(x, self.weight, out, self.algo)
            return out
        if self.overlap_class.get_option("mode") == 1:
            if self._tmp is None or self._tmp.shape != (x.size(0), N):
                self._tmp = torch.empty((x.size(0), N), dtype=x.dtype, device=x.device)
            tmp = self._tmp
        else:
            tmp = out  # the fused kernel needs no full-size scratch
        self.overlap_class.gemm_reducescatter_overlap(
            x, self.weight, tmp, out, self.counter, self.reorder_array, self.row_array, 1, self.cseg_cpu,
            self.cseg_gpu, self.algo, False)
        return out
