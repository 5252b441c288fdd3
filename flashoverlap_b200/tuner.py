"""Wave-group tuning: latency model, candidate enumeration and the two search strategies.

The reference tunes ONE mechanism - a signalling GEMM plus one NCCL call per wave group on a
second stream - with either an exhaustive timing of every grouping or a predictive search fed by
a measured NCCL bandwidth curve (tune/search.py:207-235 ``predict_lat``, :376-502).  This module
keeps both searches and the file formats, and re-derives the model for B200:

* ``mode="gated"``  - the reference's mechanism on our GEMM.  NCCL needs SMs of its own, so the
  GEMM runs on ``sm_count - sm_margin`` CTAs (the reference hard-codes ``sm_count - 2``); the
  GEMM time measured on the full machine is rescaled by the change in wave count, and groups
  pipeline against their collectives exactly as in the reference's two-stage recurrence.
* ``mode="fused"``  - the in-kernel collective.  No SM is taken from the GEMM; a group's
  reduction is done by the reducer warps of the CTAs that produced it and starts as soon as every
  rank has pushed the group, so only the tail after the last group is exposed, plus whatever the
  NVLink transfer cannot hide when the op is communication bound.

All functions here are pure (no GPU needed) except the ``measure`` callables handed in by the
CLI scripts in ``tune/``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional, Sequence, Tuple

import torch

from .utils import layout

BANDWIDTH_POINTS = 36
# Fused-mode model constants (see predict_latency)
kFusedComputeFactor = 1.05
kFusedTailMs = 0.030
kGatedCommFactor = 1.5


def bandwidth_sizes() -> List[int]:
    """Element counts of the bandwidth curve: 2**20 .. 2**28.75 in quarter-octave steps, rounded
    down to a multiple of 1024 (same sampling as the reference, tune/bandwidth.py:77)."""
    return [int(2 ** (20 + 0.25 * i)) // 1024 * 1024 for i in range(BANDWIDTH_POINTS)]


def algorithmic_bytes(elems: float, comm_op: str, world_size: int, elem_size: int = 2) -> float:
    """Bytes counted against the curve: 2(ws-1) x payload for all_reduce, (ws-1) x for
    reduce_scatter - the reference's convention (tune/bandwidth.py:88-96)."""
    factor = 2 * (world_size - 1) if comm_op == "all_reduce" else (world_size - 1)
    return elems * elem_size * factor


def curve_from_timings(sizes: Sequence[int], ms: Sequence[float], comm_op: str, world_size: int) -> torch.Tensor:
    """[len, 2] tensor of (elements, GiB per millisecond) as stored in bandwidth_*.pt."""
    rows = []
    for n, t in zip(sizes, ms):
        rows.append([float(n), algorithmic_bytes(n, comm_op, world_size) / max(t, 1e-9) / 2 ** 30])
    return torch.tensor(rows, dtype=torch.float32)


def interpolate_bandwidth(curve: torch.Tensor, elems: float) -> float:
    """Piecewise-linear interpolation of the curve, clamped at both ends."""
    xs, ys = curve[:, 0].tolist(), curve[:, 1].tolist()
    if elems <= xs[0]:
        return ys[0]
    if elems >= xs[-1]:
        return ys[-1]
    for i in range(1, len(xs)):
        if elems <= xs[i]:
            w = (elems - xs[i - 1]) / (xs[i] - xs[i - 1])
            return ys[i - 1] + w * (ys[i] - ys[i - 1])
    return ys[-1]


def comm_latency_ms(curve: torch.Tensor, elems: float, comm_op: str, world_size: int) -> float:
    """Time of one collective over ``elems`` 16-bit elements according to the curve."""
    if elems <= 0 or world_size <= 1:
        return 0.0
    return algorithmic_bytes(elems, comm_op, world_size) / interpolate_bandwidth(curve, elems) / 2 ** 30


@dataclass
class Problem:
    M: int
    N: int
    BM: int
    BN: int
    gemm_ms: float          # plain GEMM time on the full machine
    sm_count: int
    world_size: int
    comm_op: str            # "all_reduce" | "reduce_scatter"
    sm_margin: int = 2      # SMs the GEMM leaves to NCCL in gated mode
    grid: Optional[int] = None  # CTAs of the fused launch (defaults to sm_count)

    @property
    def tiles(self) -> int:
        return (self.M // self.BM) * (self.N // self.BN)

    @property
    def tile_elems(self) -> int:
        return self.BM * self.BN


def predict_latency(p: Problem, cseg: Sequence[int], curve: torch.Tensor, mode: str = "fused") -> float:
    """Predicted latency (ms) of the overlapped op for the grouping ``cseg`` (tiles per group)."""
    if sum(cseg) != p.tiles:
        raise ValueError("sum(cSeg) must equal the number of tiles")
    comm = lambda tiles: comm_latency_ms(curve, tiles * p.tile_elems, p.comm_op, p.world_size)
    if len(cseg) == 1:
        # no overlap at all: GEMM, then one collective
        return p.gemm_ms + comm(cseg[0])
    full_grid = p.grid or p.sm_count
    if mode == "gated":
        # A collective that runs under the GEMM shares SMs, L2 and power with it.  Fitted on the
        # 72 measured groupings of the tp2 / tp4 / tp8 sweeps (exhaustive best and the model's
        # earlier pick for each of 36 cases): charging it 1.5x its stand-alone time from the curve
        # minimises the mean |error| (8.7 %; 10.7 % at 1.2x, 15.9 % at 2x); a smaller factor
        # over-segments - on B200 the exhaustive best is one or two groups in most cases.
        base_comm = comm
        comm = lambda tiles: kGatedCommFactor * base_comm(tiles)
        wave = max(1, p.sm_count - p.sm_margin)
        old_waves = layout.div_up(p.tiles, p.sm_count)
        new_waves = layout.div_up(p.tiles, wave)
        per_wave = p.gemm_ms / old_waves            # a wave costs the same on fewer SMs
        comp_of = lambda tiles: per_wave * layout.div_up(tiles, wave)
        del new_waves
    elif mode == "fused":
        # Tiles retire continuously on a persistent grid: compute time is proportional to tiles.
        # Fitted on the tp2 / tp8 sweeps (profiles/sweep_tp*.md): the fused kernel's main loop runs
        # about 5 % slower than the plain GEMM's (its epilogue feeds the push warp), the groups'
        # transfers stream back to back at the curve's ASYMPTOTIC bandwidth (a group's message is
        # not a collective call of its own: the per-call latency that the small-message end of the
        # curve contains is paid once, as the tail after the last group), and that tail - pipeline fill,
        # the last tile's reduction and the end-of-call handshake - is about 30 us.  Mean |error| of
        # the fit on the tp2 sweep: 6 %, worst 16 % (the 1024-row shapes).
        per_tile = kFusedComputeFactor * p.gemm_ms / layout.div_up(p.tiles, full_grid) / full_grid
        comp_of = lambda tiles: per_tile * tiles
        bw_inf = float(curve[:, 1].max())
        comm = lambda tiles: algorithmic_bytes(tiles * p.tile_elems, p.comm_op, p.world_size) / bw_inf / 2 ** 30
        comp_t, comm_t = 0.0, 0.0
        for i, g in enumerate(cseg):
            prev_comm = comm(cseg[i - 1]) if i > 0 else 0.0
            comm_t = max(comp_t, comm_t) + prev_comm
            comp_t += comp_of(g)
        return max(comp_t, comm_t) + comm(cseg[-1]) + kFusedTailMs
    else:
        raise ValueError("mode must be 'gated' or 'fused'")
    comp_t, comm_t = 0.0, 0.0
    for i, g in enumerate(cseg):
        prev_comm = comm(cseg[i - 1]) if i > 0 else 0.0
        comm_t = max(comp_t, comm_t) + prev_comm     # group i-1's collective runs under group i
        comp_t += comp_of(g)
    return max(comp_t, comm_t) + comm(cseg[-1])


def candidate_groupings(tiles: int, wave_size: int, max_waves_per_unit: int = 10,
                        prune_cold_start: bool = True) -> List[List[int]]:
    """All groupings the searches consider, as tiles per group.

    Waves are first merged into at most ``max_waves_per_unit`` units (the reference's
    ``min_group_size``, tune/search.py:462), every ordered composition of the unit count is a
    candidate; compositions with more than 5 groups whose first group spans more than 2 units are
    dropped when ``prune_cold_start`` (the reference's "avoid cold start" rule, :483).
    """
    waves = layout.div_up(tiles, wave_size)
    unit = layout.div_up(waves, max_waves_per_unit)
    units = layout.div_up(waves, unit)
    out = []
    for comp in layout.integer_compositions(units):
        if prune_cold_start and len(comp) > 5 and comp[0] > 2:
            continue
        cseg, acc = [], 0
        for j, c in enumerate(comp):
            n = c * unit * wave_size
            if j == len(comp) - 1 or acc + n > tiles:
                n = tiles - acc
            if n <= 0:
                break
            cseg.append(n)
            acc += n
        if sum(cseg) == tiles:
            out.append(cseg)
    # de-duplicate while keeping order
    seen, uniq = set(), []
    for c in out:
        k = tuple(c)
        if k not in seen:
            seen.add(k)
            uniq.append(c)
    return uniq


def predictive_search(p: Problem, curve: torch.Tensor, mode: str = "fused",
                      candidates: Optional[Iterable[Sequence[int]]] = None,
                      wave_size: Optional[int] = None) -> Tuple[List[int], float]:
    """Grouping with the lowest predicted latency; returns (cSeg, predicted ms)."""
    if wave_size is None:
        wave_size = (p.sm_count - p.sm_margin) if mode == "gated" else (p.grid or p.sm_count)
    if candidates is None:
        candidates = candidate_groupings(p.tiles, wave_size)
        if mode == "fused":
            candidates = list(candidates) + [[1] * p.tiles]      # one flag per tile
    best, best_t = None, math.inf
    for c in candidates:
        t = predict_latency(p, c, curve, mode)
        if t < best_t:
            best, best_t = list(c), t
    return best, best_t


def exhaustive_search(candidates: Iterable[Sequence[int]], measure: Callable[[Sequence[int]], float],
                      log: Optional[Callable[[str], None]] = None) -> Tuple[List[int], float, List[Tuple[List[int], float]]]:
    """Times every candidate with ``measure`` (ms); returns (best cSeg, best ms, all results)."""
    results = []
    best, best_t = None, math.inf
    for c in candidates:
        t = float(measure(list(c)))
        results.append((list(c), t))
        if log:
            log(f"{list(c)} {t:.4f}")
        if t < best_t:
            best, best_t = list(c), t
    return best, best_t, results


def roofline_ms(M: int, N: int, K_per_rank: int, world_size: int, comm_op: str, peak_tflops: float,
                link_gbs: float, elem_size: int = 2) -> float:
    """The slower of the GEMM at tensor-core peak and the bytes that must cross NVLink
    (per direction per GPU) at link bandwidth: S(ws-1)/ws for reduce_scatter, twice that for a
    peer-to-peer all_reduce."""
    t_gemm = 2.0 * M * N * K_per_rank / (peak_tflops * 1e12)
    S = M * N * elem_size
    factor = (2.0 if comm_op == "all_reduce" else 1.0) * (world_size - 1) / max(1, world_size)
    t_link = S * factor / (link_gbs * 1e9) if world_size > 1 else 0.0
    return max(t_gemm, t_link) * 1e3
