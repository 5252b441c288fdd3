"""Functional models of the two overlap mechanisms, in plain PyTorch.

* ``gated_*``: the reference's mechanism (src/overlap_impl.cu:214-321) - the GEMM writes its
  tiles in completion order into a tile-contiguous buffer, and each wave group's contiguous
  range is all-reduced / reduce-scattered by its own collective call.  These functions run
  under ``torch.distributed`` with any backend; the CPU tests use ``gloo`` with 2 ranks.
* ``fused_*``: the protocol of the fused sm_100a kernels - every rank pushes the row slices of
  each partial tile to the rank that owns them, the owner sums the ``world`` partials in fp32
  and writes the result to every rank (AllReduce) or keeps it (ReduceScatter).  Modelled in one
  process over lists of per-rank operands, with the same staging layout and ownership rules as
  csrc/gemm/fo_gemm_sm100.cuh, so that index arithmetic can be checked without a GPU.

Nothing here is a fast path; it is the oracle.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..utils import layout


def local_gemm(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """C = A @ B^T with fp32 accumulation, rounded to the operand dtype."""
    return (A.float() @ B.float().t()).to(A.dtype)


# ----------------------------------------------------------------------------- gated model

def gated_allreduce(A, B, BM: int, BN: int, hint: Sequence[int], cseg: Sequence[int],
                    group=None) -> torch.Tensor:
    """Returns the all-reduced output in the tile-contiguous layout (flat)."""
    M, N = A.shape[0], B.shape[0]
    RA = layout.reorder_indices((M // BM) * (N // BN), hint)
    buf = layout.to_reordered(local_gemm(A, B), BM, BN, RA).contiguous()
    for start, length in layout.group_ranges(cseg, BM * BN):
        seg = buf[start:start + length]
        dist.all_reduce(seg, group=group)          # one collective per wave group
    return buf


def gated_reducescatter(A, B, BM: int, BN: int, hint: Sequence[int], cseg: Sequence[int],
                        group=None) -> torch.Tensor:
    """Returns this rank's shard [M/ws * N] as tiles of BM/ws x BN in reordered order (flat)."""
    ws = dist.get_world_size(group)
    M, N = A.shape[0], B.shape[0]
    RA = layout.reorder_indices((M // BM) * (N // BN), hint)
    RE = layout.generate_row_mapping(M, N, BM, BN, cseg, ws).long()
    rows = layout.to_reordered(local_gemm(A, B), BM, BN, RA).reshape(-1, BN)
    scattered = torch.empty_like(rows)
    scattered[RE] = rows                            # what the scatter epilogue writes
    flat = scattered.reshape(-1)
    out = torch.empty(M * N // ws, dtype=A.dtype)
    for start, length in layout.group_ranges(cseg, BM * BN):
        send = flat[start:start + length]
        recv = out[start // ws:(start + length) // ws]
        dist.reduce_scatter_tensor(recv, send.contiguous(), group=group)
    return out


# ----------------------------------------------------------------------------- fused model

def _stage_push(stage: List[torch.Tensor], src: int, partial: torch.Tensor, BM: int, BN: int,
                ws: int, strided: bool) -> None:
    """Rank ``src`` pushes every tile's row slices into the owners' staging buffers.

    stage[o] has shape [ws, tiles, BM/ws, BN]: (source rank, natural tile id, owned row, col).
    """
    M, N = partial.shape
    tm, tn = M // BM, N // BN
    tiles = partial.reshape(tm, BM, tn, BN).permute(0, 2, 1, 3).reshape(tm * tn, BM, BN)
    rows_owned = BM // ws
    for o in range(ws):
        if strided:
            sl = tiles[:, o::ws, :]                 # local rows o, o+ws, ...
        else:
            sl = tiles[:, o * rows_owned:(o + 1) * rows_owned, :]
        stage[o][src] = sl


def fused_collective(A: List[torch.Tensor], B: List[torch.Tensor], BM: int, BN: int, comm_op: str,
                     strided: bool = True, RA: Optional[torch.Tensor] = None,
                     natural_out: bool = True) -> List[torch.Tensor]:
    """Per-rank results of the fused kernel for operands A[r] [M,K], B[r] [N,K].

    all_reduce: each entry is the full [M,N] sum (row-major if ``natural_out`` else flat
    tile-contiguous per RA).  reduce_scatter: each entry is the rank's shard - row-major
    [M/ws, N] holding its owned rows in ascending order, or flat tiles of BM/ws x BN.
    """
    ws = len(A)
    M, N = A[0].shape[0], B[0].shape[0]
    tm, tn = M // BM, N // BN
    rows_owned = BM // ws
    dt = A[0].dtype
    if RA is None:
        RA = torch.arange(tm * tn, dtype=torch.int32)
    stage = [torch.zeros(ws, tm * tn, rows_owned, BN, dtype=dt) for _ in range(ws)]
    for r in range(ws):
        _stage_push(stage, r, local_gemm(A[r], B[r]), BM, BN, ws, strided)
    # owner o: fp32 sum over sources, one rounding
    reduced = [stage[o].float().sum(0).to(dt) for o in range(ws)]   # [tiles, rows_owned, BN]
    outs = []
    if comm_op == "all_reduce":
        tiles = torch.empty(tm * tn, BM, BN, dtype=dt)
        for o in range(ws):
            if strided:
                tiles[:, o::ws, :] = reduced[o]
            else:
                tiles[:, o * rows_owned:(o + 1) * rows_owned, :] = reduced[o]
        full = tiles.reshape(tm, tn, BM, BN).permute(0, 2, 1, 3).reshape(M, N)
        for _ in range(ws):
            outs.append(full.clone() if natural_out else layout.to_reordered(full, BM, BN, RA))
        return outs
    if comm_op == "reduce_scatter":
        for o in range(ws):
            shard = reduced[o].reshape(tm, tn, rows_owned, BN).permute(0, 2, 1, 3).reshape(M // ws, N)
            outs.append(shard if natural_out else layout.to_reordered(shard, rows_owned, BN, RA))
        return outs
    raise ValueError("comm_op must be 'all_reduce' or 'reduce_scatter'")
