"""Per-tile timeline of the fused GEMM+collective kernels.

``OverlapImpl.set_trace(buf)`` (or ``ops.fused_loopback(..., trace=buf)``) makes the fused
AllReduce / ReduceScatter kernels stamp, for every 128-row output tile, eight 64-bit words
(nanoseconds of the GPU's global timer; layout ``TraceSlot`` in csrc/gemm/fo_gemm_params.h):

    0 acc_ready       the tile's accumulator is complete (main loop done)
    1 epilogue_done   last chunk handed to the push warp
    2 push_issued     last store of the tile issued towards the owners
    3 signalled       the stores have completed and the owners' arrival counters are bumped
    4 wait_begin      the owner's reducer starts waiting for the tile
    5 wait_end        every rank's slice has arrived
    6 reduced         the reduction of the tile has been issued completely
    7 where           (SM id << 32) | CTA index

Slots 0-3 are written by the rank that computed the tile, 4-6 by its reducer on the same rank
(every rank runs the same tile schedule, so the CTA that computes a tile also reduces this
rank's slice of it).  The reference has no timeline beyond a profiler screenshot
(docs/_static/image/typical_timeline.jpeg); this is the in-library substitute.
"""
from __future__ import annotations

import json
from typing import Dict, List

import torch

SLOTS = 8
NAMES = ["acc_ready", "epilogue_done", "push_issued", "signalled", "wait_begin", "wait_end", "reduced", "where"]
# (name, from slot, to slot)
PHASES = [("epilogue", 0, 1), ("push_issue", 1, 2), ("push_complete", 2, 3), ("arrival_wait", 4, 5), ("reduce", 5, 6),
          ("acc_ready_to_reduced", 0, 6)]


def new_buffer(tiles: int, ranks: int = 1, device="cuda") -> torch.Tensor:
    return torch.zeros(ranks * tiles * SLOTS, dtype=torch.int64, device=device)


def _table(buf: torch.Tensor, tiles: int, rank: int = 0) -> torch.Tensor:
    t = buf.detach().cpu().reshape(-1, SLOTS)
    return t[rank * tiles:(rank + 1) * tiles]


def summarize(buf: torch.Tensor, tiles: int, rank: int = 0) -> Dict[str, Dict[str, float]]:
    """Mean / median / max duration (microseconds) of every phase over the tiles that were
    stamped, plus the span from the first accumulator to the last reduction."""
    t = _table(buf, tiles, rank)
    out: Dict[str, Dict[str, float]] = {}
    for name, a, b in PHASES:
        ok = (t[:, a] > 0) & (t[:, b] > 0)
        if not ok.any():
            continue
        d = (t[ok, b] - t[ok, a]).double() / 1e3
        out[name] = {"mean_us": float(d.mean()), "median_us": float(d.median()), "max_us": float(d.max()),
                     "tiles": int(ok.sum())}
    stamped = t[:, :7][t[:, :7] > 0]
    if stamped.numel():
        out["span"] = {"us": float((stamped.max() - stamped.min()).double() / 1e3)}
    return out


def to_chrome_trace(buf: torch.Tensor, tiles: int, path: str, rank: int = 0) -> List[dict]:
    """Writes a Chrome / Perfetto trace (JSON): one process per rank, one thread per CTA and
    role, one slice per tile and phase.  Returns the events."""
    t = _table(buf, tiles, rank)
    stamped = t[:, :7][t[:, :7] > 0]
    origin = int(stamped.min()) if stamped.numel() else 0
    roles = {"epilogue": 0, "push_issue": 1, "push_complete": 1, "arrival_wait": 2, "reduce": 2}
    role_names = ["epilogue", "push", "reducer"]
    events: List[dict] = []
    seen = set()
    for tile in range(tiles):
        row = t[tile]
        cta = int(row[7]) & 0xFFFFFFFF
        sm = int(row[7]) >> 32
        for name, a, b in PHASES[:5]:
            if row[a] <= 0 or row[b] <= 0:
                continue
            tid = cta * 4 + roles[name]
            if tid not in seen:
                seen.add(tid)
                events.append({"ph": "M", "name": "thread_name", "pid": rank, "tid": tid,
                               "args": {"name": f"cta {cta} (sm {sm}) {role_names[roles[name]]}"}})
            events.append({"ph": "X", "name": name, "cat": "tile", "pid": rank, "tid": tid,
                           "ts": (int(row[a]) - origin) / 1e3, "dur": max(0.0, (int(row[b]) - int(row[a])) / 1e3),
                           "args": {"tile": tile}})
    with open(path, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ns"}, f)
    return events
