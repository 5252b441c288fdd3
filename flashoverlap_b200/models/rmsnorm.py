"""RMSNorm modules (reference: example/RMSNorm.py:7-33).

``RMSNorm`` is the plain PyTorch reference module; with ``fused=True`` it calls the sm_100a
row kernel instead.  ``ReorderRMSNorm`` consumes the tile-contiguous buffer produced by the
overlapped GEMM and returns the row-major, normalised result in one pass over memory.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.nn as nn

from ..utils import layout


def _default_device():
    return "cuda" if torch.cuda.is_available() else "cpu"


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, dtype=torch.bfloat16, device=None, fused: bool = False):
        super().__init__()
        self.eps = eps
        self.fused = fused
        self.weight = nn.Parameter(
            torch.empty(dim, dtype=dtype, device=device or _default_device()).normal_(mean=1.0, std=0.02))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.fused and x.is_cuda:
            from .._build import load
            load()
            x2 = x.reshape(-1, x.shape[-1]).contiguous()
            out = torch.empty_like(x2)
            torch.ops.flashoverlap_op.rmsnorm(x2, out, self.weight, self.eps)
            return out.view_as(x)
        return layout.rmsnorm_ref(x, self.weight, self.eps)


class ReorderRMSNorm(nn.Module):
    """Un-reorder + RMSNorm.  ``M`` is the number of rows of the buffer this module will see
    (``M // world`` with ``BM // world``-row tiles after a reduce-scatter)."""

    def __init__(self, dim: int, M: int, BM: int, BN: int, hint: Sequence[int], eps: float = 1e-6,
                 dtype=torch.bfloat16, device=None):
        super().__init__()
        device = device or _default_device()
        self.eps = eps
        self.bm, self.bn = BM, BN
        self.weight = nn.Parameter(torch.empty(dim, dtype=dtype, device=device).normal_(mean=1.0, std=0.02))
        tm, tn = layout.div_up(M, BM), layout.div_up(dim, BN)
        self.register_buffer("reorder_array",
                             layout.reorder_indices(tm * tn, hint, device=device).reshape(tm, tn),
                             persistent=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rows, dim = x.shape[0], x.shape[1]
        if x.is_cuda:
            from .._build import load
            load()
            out = torch.empty((rows, dim), dtype=x.dtype, device=x.device)
            torch.ops.flashoverlap_op.reorder_rmsnorm_eps(x, out, self.weight, self.bm, self.bn, 1,
                                                          self.reorder_array, self.eps)
            return out
        return layout.reorder_rmsnorm_ref(x, rows, dim, self.bm, self.bn, self.reorder_array,
                                          self.weight, self.eps)
