"""Tile orders, the tile-contiguous ("reordered") layout and the reduce-scatter row maps.

Pure PyTorch, runs on CPU: this module is the executable specification every kernel is tested
against.  It covers what the reference keeps in ``example/utils.py`` (``reorder_indices`` :6-22,
``generate_row_mapping`` :24-52, ``reorder_rows_by_world_size`` :54-65; copies of the first two
also live in test/test.py:23-69 and tune/search.py:53-81,237-253) plus the layout rules that the
reference only implements inside its CUDA epilogue (src/overlap/gemm_with_signal.h:236-256) and
norm kernel (src/rmsnorm/rmsnorm.cuh:80-86).

Vocabulary: the output [M, N] is cut into TM x TN tiles of BM x BN; the *natural* id of tile
(i, j) is ``i * TN + j``; ``RA[natural id]`` is the tile's *position* in the reordered buffer,
where tiles are stored one after another, each as BM contiguous rows of BN elements
(``rLDN`` > 1 puts that many tiles side by side).  ``hint`` lists natural ids in the order the
GEMM finishes them, so ``RA = reorder_indices(TM*TN, hint)`` makes completion order ==
memory order, and a *wave group* (``cSeg[g]`` consecutive positions) is one contiguous range.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

import torch


def div_up(x: int, y: int) -> int:
    return (x + y - 1) // y


# ----------------------------------------------------------------------------- tile orders

def raster_order(tiles_m: int, tiles_n: int, strip: int, rows_per_unit: int = 1) -> List[int]:
    """Natural tile ids in the order the persistent GEMM visits them.

    ``rows_per_unit``: the CTA-pair kernels schedule units of 2 (or, with two row halves per CTA,
    4) vertically adjacent 128-row tiles that are produced together; they are listed top to
    bottom.  ``True`` is accepted for 2.

    Tiles are swept in column strips ``strip`` tiles wide, M-major inside a strip
    (``strip <= 0`` or ``>= tiles_n``: full row panels).  Mirrors ``tile_of_position`` in
    csrc/gemm/fo_gemm_sm100.cuh; the counterpart of CUTLASS's threadblock swizzle in the
    reference (src/overlap/gemm_with_epilogue_visitor.h:316-326).
    """
    if strip <= 0 or strip > tiles_n:
        strip = tiles_n
    g = 2 if rows_per_unit is True else max(1, int(rows_per_unit))
    if tiles_m % g:
        raise ValueError("the number of tile rows must be a multiple of the rows per scheduling unit")
    order: List[int] = []
    sched_m = tiles_m // g
    for s in range(div_up(tiles_n, strip)):
        w = min(strip, tiles_n - s * strip)
        for m in range(sched_m):
            for j in range(w):
                n = s * strip + j
                for i in range(g):
                    order.append((g * m + i) * tiles_n + n)
    return order


def analytic_hint(M: int, N: int, BM: int, BN: int, strip: int, rows_per_unit: int = 1) -> List[int]:
    """Completion-order hint of the persistent kernel, known by construction.

    CTA c of a grid of G processes positions c, c+G, ... of ``raster_order``; wave w is the
    positions [w*G, (w+1)*G).  The reference has to measure this order with a monitor run
    because its tiles are dispatched by the hardware block scheduler (tune/search.py:83-178).
    """
    return raster_order(M // BM, N // BN, strip, rows_per_unit)


def reorder_indices(num_tiles: int, hint: Sequence[int], device="cpu") -> torch.Tensor:
    """RA with ``RA[hint[p]] = p``; tiles missing from ``hint`` follow in ascending id order."""
    hint_t = torch.as_tensor(list(hint), dtype=torch.long)
    if hint_t.numel() and (hint_t.min() < 0 or hint_t.max() >= num_tiles):
        raise ValueError("hint contains an id outside [0, num_tiles)")
    if hint_t.unique().numel() != hint_t.numel():
        raise ValueError("hint contains duplicate tile ids")
    seen = torch.zeros(num_tiles, dtype=torch.bool)
    seen[hint_t] = True
    rest = torch.nonzero(~seen).flatten()
    order = torch.cat([hint_t, rest])
    ra = torch.empty(num_tiles, dtype=torch.int32)
    ra[order] = torch.arange(num_tiles, dtype=torch.int32)
    return ra.to(device)


def generate_row_mapping(M: int, N: int, BM: int, BN: int, cseg: Sequence[int], world_size: int,
                         device="cpu") -> torch.Tensor:
    """RE for the counter-gated reduce-scatter: ``RE[row] = new row`` of the [M*N/BN, BN] view.

    Inside each wave group's row range the rows are stably sorted by ``row % world_size``, so a
    plain reduce-scatter over the group's contiguous range hands rank p exactly the rows
    congruent to p.
    """
    total_tiles = (M * N) // (BM * BN)
    if sum(cseg) != total_tiles:
        raise ValueError("sum(cSeg) must equal the number of tiles")
    rows = torch.arange(M * N // BN, dtype=torch.long)
    new_of_old = torch.empty_like(rows)
    start = 0
    for s in cseg:
        n = s * BM
        chunk = rows[start:start + n]
        key = chunk % world_size
        perm = torch.sort(key, stable=True).indices          # position -> source offset in chunk
        new_of_old[chunk[perm]] = torch.arange(start, start + n)
        start += n
    return new_of_old.to(torch.int32).to(device)


def reorder_rows_by_world_size(x: torch.Tensor, world_size: int) -> torch.Tensor:
    """Rows grouped by ``row % world_size`` (stable): rank p's shard is the p-th block."""
    idx = torch.arange(x.shape[0], device=x.device)
    perm = torch.sort(idx % world_size, stable=True).indices
    return x[perm]


def owned_rows(M: int, BM: int, world_size: int, rank: int, strided: bool = True) -> torch.Tensor:
    """Logical row indices a rank receives from the fused reduce-scatter, ascending.

    strided: rows with ``row % world_size == rank`` (the reference's ownership);
    otherwise each tile's rows are split into contiguous blocks of BM/world_size rows.
    """
    idx = torch.arange(M)
    if strided:
        return idx[(idx % BM) % world_size == rank]
    return idx[(idx % BM) // (BM // world_size) == rank]


def gathered_as_tokens(buf: torch.Tensor, world_size: int, BM: int = 128) -> torch.Tensor:
    """Token-ordered VIEW of an all-gathered matrix whose shards follow the contiguous-block
    ownership of the fused reduce-scatter (``owned_rows(..., strided=False)``).

    ``buf`` is ``[world_size * n, c]`` in gather order (rank-major).  Rank r's shard holds rows
    ``r*BM/ws .. (r+1)*BM/ws - 1`` of every BM-row tile, so token ``tile*BM + r*BM/ws + i`` sits at
    ``buf[r*n + tile*BM/ws + i]``.  The result has shape ``[tiles, world_size, BM/ws, c]`` and is
    not contiguous: ``.reshape(-1, c)`` copies it into token order, and as the ``out=`` of an
    elementwise op over rank-major inputs it places their result in token order without a pass
    of its own (give it a token-ordered buffer and use the result of
    ``gathered_as_tokens(buffer.view_as(rank_major), ...)`` the other way round, see
    ``tokens_as_gathered``)."""
    rows, c = buf.shape
    n, ro = rows // world_size, BM // world_size
    return buf.view(world_size, n // ro, ro, c).permute(1, 0, 2, 3)


def tokens_as_gathered(buf: torch.Tensor, world_size: int, BM: int = 128) -> torch.Tensor:
    """The inverse view: a token-ordered ``[T, c]`` matrix indexed ``[rank, tile, row in block, c]``,
    i.e. in the order an all-gather of the ranks' shards delivers."""
    rows, c = buf.shape
    ro = BM // world_size
    return buf.view(rows // BM, world_size, ro, c).permute(1, 0, 2, 3)


# ----------------------------------------------------------------------------- layouts

def _tile_offsets(M, N, BM, BN, RA, rldn):
    tm, tn = M // BM, N // BN
    ra = torch.as_tensor(RA, dtype=torch.long).flatten().cpu()
    if ra.numel() < tm * tn:
        raise ValueError("RA has fewer entries than there are tiles")
    return tm, tn, ra


def to_reordered(C: torch.Tensor, BM: int, BN: int, RA, rldn: int = 1) -> torch.Tensor:
    """Flat tile-contiguous copy of row-major ``C`` (what the GEMM epilogue writes)."""
    M, N = C.shape
    tm, tn, ra = _tile_offsets(M, N, BM, BN, RA, rldn)
    tiles = C.reshape(tm, BM, tn, BN).permute(0, 2, 1, 3).reshape(tm * tn, BM, BN)
    if rldn == 1:
        out = torch.empty_like(tiles)
        out[ra.to(C.device)] = tiles
        return out.reshape(-1)
    # rldn tiles side by side: reordered matrix has M*N/(rldn*BN) rows of rldn*BN columns
    if (tm * tn) % rldn:
        raise ValueError("rLDN must divide the tile count")
    out = torch.empty((tm * tn) // rldn, BM, rldn, BN, dtype=C.dtype, device=C.device)
    r = ra.to(C.device)
    out[r // rldn, :, r % rldn, :] = tiles
    return out.reshape(-1)


def from_reordered(buf: torch.Tensor, M: int, N: int, BM: int, BN: int, RA, rldn: int = 1) -> torch.Tensor:
    """Row-major [M, N] matrix recovered from the tile-contiguous buffer."""
    tm, tn, ra = _tile_offsets(M, N, BM, BN, RA, rldn)
    r = ra.to(buf.device)
    flat = buf.reshape(-1)[: M * N]
    if rldn == 1:
        tiles = flat.reshape(tm * tn, BM, BN)[r]
    else:
        tiles = flat.reshape((tm * tn) // rldn, BM, rldn, BN)[r // rldn, :, r % rldn, :]
    return tiles.reshape(tm, tn, BM, BN).permute(0, 2, 1, 3).reshape(M, N)


def rmsnorm_ref(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 normalisation, cast back to x's dtype, then times weight (example/RMSNorm.py:7-18)."""
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return n.to(x.dtype) * weight


def reorder_rmsnorm_ref(buf: torch.Tensor, rows: int, dim: int, BM: int, BN: int, RA,
                        weight: torch.Tensor, eps: float, rldn: int = 1) -> torch.Tensor:
    """Oracle of the fused un-reorder + RMSNorm kernel."""
    return rmsnorm_ref(from_reordered(buf, rows, dim, BM, BN, RA, rldn), weight, eps)


# ----------------------------------------------------------------------------- wave groups

def waves_of(num_tiles: int, wave_size: int) -> List[int]:
    """Tiles per wave when ``wave_size`` CTAs each take one tile per wave."""
    full, rem = divmod(num_tiles, wave_size)
    return [wave_size] * full + ([rem] if rem else [])


def cseg_from_wave_groups(num_tiles: int, wave_size: int, groups: Sequence[int]) -> List[int]:
    """Tiles per wave group for a partition ``groups`` of the wave count (sum == #waves)."""
    waves = waves_of(num_tiles, wave_size)
    if sum(groups) != len(waves):
        raise ValueError("group sizes must add up to the number of waves")
    out, i = [], 0
    for g in groups:
        out.append(sum(waves[i:i + g]))
        i += g
    return out


def group_ranges(cseg: Sequence[int], tile_elems: int) -> List[tuple]:
    """(start, length) in elements of each wave group's contiguous range."""
    out, acc = [], 0
    for s in cseg:
        out.append((acc * tile_elems, s * tile_elems))
        acc += s
    return out


def integer_compositions(n: int, max_parts: Optional[int] = None) -> Iterable[List[int]]:
    """All ordered ways to write n as a sum of positive integers (2**(n-1) of them)."""
    if n == 0:
        yield []
        return

    def rec(rest, parts):
        if rest == 0:
            yield list(parts)
            return
        if max_parts is not None and len(parts) >= max_parts:
            return
        for first in range(1, rest + 1):
            parts.append(first)
            yield from rec(rest - first, parts)
            parts.pop()

    yield from rec(n, [])


def all2all_reference(C_per_rank, mlen):
    """CPU/torch oracle of the variable-size all-to-all on packed rows (the reference's
    semantics, src/overlap_impl.cu:181-212): ``C_per_rank[r]`` holds rank r's rows, the runs for
    the other ranks packed in rank order (``mlen[r][i]`` rows for rank i, own run absent);
    returns the receive buffers, where rank i finds the runs of the other ranks in rank order."""
    ws = len(C_per_rank)
    send_off = [[0] * ws for _ in range(ws)]
    for r in range(ws):
        acc = 0
        for i in range(ws):
            send_off[r][i] = acc
            if i != r:
                acc += int(mlen[r][i])
    out = []
    for i in range(ws):
        parts = [C_per_rank[r][send_off[r][i]:send_off[r][i] + int(mlen[r][i])] for r in range(ws) if r != i]
        out.append(torch.cat(parts, 0) if parts else C_per_rank[i][:0])
    return out
