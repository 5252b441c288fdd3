"""Latency model, candidate enumeration and search drivers of the wave-group tuner (CPU)."""

import pytest
import torch

from flashoverlap_b200 import tuner
from flashoverlap_b200.utils import layout


def _flat_curve(gib_per_ms):
    sizes = tuner.bandwidth_sizes()
    return torch.tensor([[float(s), gib_per_ms] for s in sizes])


def test_bandwidth_sizes_and_curve():
    s = tuner.bandwidth_sizes()
    assert len(s) == 36 and s[0] == 2 ** 20 and all(x % 1024 == 0 for x in s) and s == sorted(s)
    assert s[-1] == int(2 ** 28.75) // 1024 * 1024
    c = tuner.curve_from_timings([2 ** 20, 2 ** 21], [1.0, 1.0], "all_reduce", 4)
    # 2^20 elements * 2 B * 2*(4-1) / 1 ms / 2^30
    assert c[0, 1].item() == pytest.approx(2 ** 20 * 2 * 6 / 2 ** 30)
    assert tuner.interpolate_bandwidth(c, 2 ** 19) == pytest.approx(c[0, 1].item())       # clamped
    mid = tuner.interpolate_bandwidth(c, 1.5 * 2 ** 20)
    assert c[0, 1].item() < mid < c[1, 1].item()
    assert tuner.comm_latency_ms(c, 2 ** 20, "all_reduce", 4) == pytest.approx(1.0)
    assert tuner.comm_latency_ms(c, 2 ** 20, "reduce_scatter", 1) == 0.0


def test_predict_latency_gated_matches_hand_computation():
    # 146-tile waves (148 SMs - 2), 4 waves of compute at 1 ms per wave (gemm 4 ms over 4 waves)
    p = tuner.Problem(M=128 * 584, N=256, BM=128, BN=256, gemm_ms=4.0, sm_count=148, world_size=2,
                      comm_op="all_reduce", sm_margin=2)
    assert p.tiles == 584 and layout.div_up(584, 148) == 4 and layout.div_up(584, 146) == 4
    curve = _flat_curve(1.0)
    per_tile = tuner.comm_latency_ms(curve, p.tile_elems, "all_reduce", 2)
    # one group: no overlap
    assert tuner.predict_latency(p, [584], curve, "gated") == pytest.approx(4.0 + 584 * per_tile)
    # two groups of two waves: comm of group 0 hides under compute of group 1; a collective that
    # runs beside the GEMM is charged kGatedCommFactor times its stand-alone time
    per_tile *= tuner.kGatedCommFactor
    c = 292 * per_tile
    expect = max(4.0, 2.0 + c) + c
    assert tuner.predict_latency(p, [292, 292], curve, "gated") == pytest.approx(expect)
    # four groups: two-stage pipeline recurrence
    c1 = 146 * per_tile
    comp, comm = 0.0, 0.0
    for i in range(4):
        comm = max(comp, comm) + (c1 if i else 0.0)
        comp += 1.0
    assert tuner.predict_latency(p, [146] * 4, curve, "gated") == pytest.approx(max(comp, comm) + c1)
    with pytest.raises(ValueError):
        tuner.predict_latency(p, [100, 100], curve, "gated")


def test_predict_latency_fused_prefers_fine_groups_when_compute_bound():
    p = tuner.Problem(M=8192, N=8192, BM=128, BN=256, gemm_ms=0.4, sm_count=148, world_size=8,
                      comm_op="all_reduce")
    curve = _flat_curve(0.9)      # ~ 0.97 TB/s algorithmic
    coarse = tuner.predict_latency(p, [p.tiles], curve, "fused")
    waves = tuner.predict_latency(p, layout.cseg_from_wave_groups(p.tiles, 148, [1] * layout.div_up(p.tiles, 148)),
                                  curve, "fused")
    fine = tuner.predict_latency(p, [1] * p.tiles, curve, "fused")
    assert fine < waves < coarse
    best, t = tuner.predictive_search(p, curve, "fused")
    assert best == [1] * p.tiles and t == pytest.approx(fine)


def test_candidate_groupings_cover_compositions_and_prune():
    cands = tuner.candidate_groupings(tiles=584, wave_size=146, prune_cold_start=False)
    assert len(cands) == 2 ** 3 and all(sum(c) == 584 for c in cands)
    assert [584] in cands and [146] * 4 in cands
    many = tuner.candidate_groupings(tiles=146 * 8, wave_size=146)
    assert all(not (len(c) > 5 and c[0] > 2 * 146) for c in many)
    # more than 10 waves are merged into units
    big = tuner.candidate_groupings(tiles=146 * 30, wave_size=146)
    assert all(sum(c) == 146 * 30 for c in big) and all(x % (3 * 146) == 0 for c in big for x in c[:-1])
    # a last partial wave is absorbed by the last group
    part = tuner.candidate_groupings(tiles=300, wave_size=146, prune_cold_start=False)
    assert [146, 146, 8] in part and [146, 154] in part


def test_exhaustive_search_picks_minimum():
    cands = [[4], [2, 2], [1, 3]]
    cost = {(4,): 3.0, (2, 2): 1.5, (1, 3): 2.0}
    seen = []
    best, t, allr = tuner.exhaustive_search(cands, lambda c: cost[tuple(c)], log=seen.append)
    assert best == [2, 2] and t == 1.5 and len(allr) == 3 and len(seen) == 3


def test_roofline():
    # AR tp=8 8192x8192x3584: GEMM-bound against 1590 TFLOP/s, link-bound against a slow link
    t = tuner.roofline_ms(8192, 8192, 3584, 8, "all_reduce", 1590.0, 770.0)
    gemm = 2 * 8192 * 8192 * 3584 / 1590e12 * 1e3
    link = 2 * 8192 * 8192 * 2 * 7 / 8 / 770e9 * 1e3
    assert t == pytest.approx(max(gemm, link))
    assert tuner.roofline_ms(128, 256, 64, 1, "all_reduce", 1590.0, 770.0) == pytest.approx(2 * 128 * 256 * 64 / 1590e12 * 1e3)
