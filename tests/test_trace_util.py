"""Timeline post-processing on a synthetic buffer (no GPU)."""
import json

import torch

from flashoverlap_b200.utils import trace


def _synthetic(tiles):
    buf = torch.zeros(tiles * trace.SLOTS, dtype=torch.int64)
    t = buf.view(tiles, trace.SLOTS)
    for i in range(tiles):
        base = 1_000_000 + 10_000 * i
        t[i, :7] = torch.tensor([base, base + 2000, base + 2500, base + 6000, base + 2100, base + 6500, base + 8000])
        t[i, 7] = (7 << 32) | (i % 3)
    return buf


def test_summary_durations():
    s = trace.summarize(_synthetic(6), 6)
    assert abs(s["epilogue"]["mean_us"] - 2.0) < 1e-9
    assert abs(s["push_complete"]["max_us"] - 3.5) < 1e-9
    assert abs(s["arrival_wait"]["median_us"] - 4.4) < 1e-9
    assert abs(s["reduce"]["mean_us"] - 1.5) < 1e-9
    assert s["epilogue"]["tiles"] == 6
    assert abs(s["span"]["us"] - (50_000 + 8000) / 1e3) < 1e-9


def test_unstamped_tiles_are_ignored(tmp_path):
    buf = _synthetic(4)
    buf.view(4, trace.SLOTS)[2] = 0
    assert trace.summarize(buf, 4)["epilogue"]["tiles"] == 3
    ev = trace.to_chrome_trace(buf, 4, str(tmp_path / "t.json"))
    slices = [e for e in ev if e["ph"] == "X"]
    assert len(slices) == 3 * 5 and all(e["dur"] >= 0 for e in slices)
    assert min(e["ts"] for e in slices) == 0.0
    assert json.load(open(tmp_path / "t.json"))["traceEvents"]
    names = {e["args"]["name"] for e in ev if e["ph"] == "M"}
    assert "cta 0 (sm 7) epilogue" in names and "cta 1 (sm 7) reducer" in names
