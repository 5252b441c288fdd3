"""Python-side handles on the native ops.

Every function here goes to a hand-written sm_100a kernel through ``torch.ops.flashoverlap_op``
(csrc/binding.cpp).  There is no PyTorch fallback for CUDA tensors: if the extension cannot
be loaded the call raises, so a GPU run can never silently measure eager code.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .._build import load as _load


def _op():
    _load()
    return torch.ops.flashoverlap_op


def OverlapImpl():
    _load()
    return torch.classes.flashoverlap_class.OverlapImpl()


def BaselineImpl():
    _load()
    return torch.classes.flashoverlap_class.BaselineImpl()


def generate_nccl_id() -> List[int]:
    return list(_op().generate_nccl_id())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, out: Optional[torch.Tensor] = None):
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    out = torch.empty_like(x2) if out is None else out
    _op().rmsnorm(x2, out, weight, eps)
    return out.view(x.shape)


def reorder_rmsnorm(x_reordered: torch.Tensor, rows: int, dim: int, weight: torch.Tensor, BM: int, BN: int,
                    RA: torch.Tensor, eps: float = 1e-5, rldn: int = 1, out: Optional[torch.Tensor] = None):
    out = torch.empty((rows, dim), dtype=x_reordered.dtype, device=x_reordered.device) if out is None else out
    _op().reorder_rmsnorm_eps(x_reordered, out, weight, BM, BN, rldn, RA, eps)
    return out


def reorder(x: torch.Tensor, BM: int, BN: int, RA: torch.Tensor, rldn: int = 1, out: Optional[torch.Tensor] = None):
    """Row-major [rows, dim] -> tile-contiguous buffer (tile t at position RA[t])."""
    out = torch.empty_like(x) if out is None else out
    _op().reorder(x.contiguous(), out, BM, BN, rldn, RA)
    return out


def unreorder(x_reordered: torch.Tensor, rows: int, dim: int, BM: int, BN: int, RA: torch.Tensor, rldn: int = 1,
              out: Optional[torch.Tensor] = None):
    out = torch.empty((rows, dim), dtype=x_reordered.dtype, device=x_reordered.device) if out is None else out
    _op().unreorder(x_reordered, out, BM, BN, rldn, RA)
    return out


def wait_flag(target: int, counters: torch.Tensor, index: int, timeout_ms: int, status: torch.Tensor) -> None:
    _op().wait_flag(target, counters, index, timeout_ms, status)


def algo_table() -> List[Sequence[int]]:
    flat = list(_op().algo_table())
    return [tuple(flat[i:i + 7]) for i in range(0, len(flat), 7)]


def fused_loopback(comm_op: str, A: List[torch.Tensor], B: List[torch.Tensor], out: List[torch.Tensor],
                   RA: Optional[torch.Tensor] = None, cseg: Optional[torch.Tensor] = None, algo: int = 0,
                   strided_rows: bool = True, natural_out: bool = True, repeat: int = 1,
                   timeout_ms: int = 1000, stage_local: bool = False,
                   mlen: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                   norm_eps: float = 1e-5, trace: Optional[torch.Tensor] = None,
                   epi_bufs: int = 2, pull_direct: bool = False,
                   norm_res: Optional[List[torch.Tensor]] = None,
                   norm_out: Optional[List[torch.Tensor]] = None) -> List[List[int]]:
    """All ranks of a fused GEMM+collective on ONE GPU in one cooperative launch (test aid).

    ``stage_local`` selects the pull protocol: every rank stages its partial tiles in its own
    memory and the owners fetch them (one load per rank here; one switch-side reduction per
    vector on a multi-GPU run whose staging has a multicast mapping).  ``comm_op="all_to_all"``
    runs the GEMM whose epilogue stores each row into its destination rank's receive buffer
    ``out[r]``; ``mlen`` is the int32 host matrix of row counts [ranks, ranks].  ``norm_w`` (with
    ``comm_op="reduce_scatter"`` and ``natural_out``) turns on the RMSNorm tail of the reducers.
    ``trace`` (int64 CUDA tensor, ranks * tiles * 8) receives the per-tile timeline, see
    ``flashoverlap_b200.utils.trace``.  ``epi_bufs=4`` runs the build with four epilogue chunk buffers.
    ``pull_direct`` (with ``stage_local``): the epilogue threads store the partial tiles into the local
    staging themselves instead of handing every chunk to the push warp's TMA stores.  ``norm_res`` /
    ``norm_out`` (with ``norm_w``): per-rank residual added to the reduced rows before they are stored in
    ``out[r]`` and normalised, and per-rank destination of the normalised rows (default: over ``out[r]``)."""
    flat = list(_op().fused_loopback(comm_op, A, B, out, RA, cseg, algo, strided_rows, natural_out, repeat,
                                     timeout_ms, stage_local, mlen, norm_w, norm_eps, trace, epi_bufs, int(pull_direct), norm_res, norm_out))
    return [flat[i:i + 8] for i in range(0, len(flat), 8)]
