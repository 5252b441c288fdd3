"""Failure detection on the host, with CPU (gloo) ranks only - no GPU is faulted or hung.

* a rank that raises before a collective must not leave its peers (or the parent) waiting;
* a rank that never joins a collective makes the others fail with a process-group timeout;
* the device status words turn into a Python exception with a readable message.
"""
import datetime
import time

import pytest
import torch
import torch.distributed as dist

from flashoverlap_b200.parallel.launch import run_on_all_gpus
from tests._mp import run_ranks


def _raises_on_rank1(rank, world):
    if rank == 1:
        raise ValueError("rank 1 fails before joining the collective")
    x = torch.ones(4)
    dist.all_reduce(x)          # would wait for rank 1 forever
    return x.sum().item()


def test_launcher_reports_failed_rank_instead_of_hanging():
    t = time.time()
    with pytest.raises(Exception):
        run_on_all_gpus(_raises_on_rank1, nprocs=2, backend="gloo")
    assert time.time() - t < 60


def _healthy(rank, world):
    x = torch.full((4,), float(rank + 1))
    dist.all_reduce(x)
    return x[0].item()


def test_launcher_returns_rank0_result():
    assert run_on_all_gpus(_healthy, nprocs=2, backend="gloo") == 3.0


def _never_joins(rank, world):
    # rank 1 sits out the collective (between steps, nothing in flight); rank 0's wait is bounded
    if rank == 1:
        time.sleep(6)
        return "skipped"
    x = torch.ones(4)
    try:
        work = dist.all_reduce(x, async_op=True)
        work.wait(timeout=datetime.timedelta(seconds=2))
        return "completed"
    except Exception as ex:          # gloo raises a timeout error
        return "timeout:" + type(ex).__name__


def test_missing_rank_is_detected_by_timeout():
    # the helper's closing barrier fails too once rank 0 has given up, so only the
    # outcome recorded before it matters
    try:
        res = run_ranks(_never_joins, 2, "gloo", timeout_s=15)
    except AssertionError as ex:
        assert "rank failure" in str(ex)
        return
    assert res[0].startswith("timeout") and res[1] == "skipped"


def test_status_words_become_exception(lib):
    """Host side of device failure reporting, without a device: the text check_status() raises for
    every status code a kernel can record, with its three diagnostic words and the rank."""
    msg = torch.ops.flashoverlap_op.status_message
    assert msg([0] * 8, 0) == ""
    expect = {1: "MMA warp waiting for TMA stage", 2: "TMA warp waiting for free stage",
              3: "epilogue waiting for accumulator", 4: "MMA warp waiting for free accumulator",
              5: "reducer waiting for peers' tile/group flag", 6: "end-of-call handshake",
              7: "start-of-call handshake", 8: "counting wait kernel", 9: "bad argument"}
    for code, text in expect.items():
        m = msg([code, 11, 22, 33, 0, 0, 0, 0], 5)
        assert text in m and "(args 11, 22, 33)" in m and m.endswith("on rank 5"), m
        assert ("timeout" in m) == (code <= 8)
    assert "unknown" in msg([77, 0, 0, 0, 0, 0, 0, 0], 0)
    with pytest.raises(RuntimeError, match="status block"):
        msg([1, 2], 0)


def test_rank_runner_retries_on_a_taken_rendezvous_port(monkeypatch):
    """The helper that runs test ranks picks its port by bind-and-close, so the port can be
    taken before rank 0 listens on it; such a run is repeated on a fresh port, other failures
    are not."""
    from tests import _mp
    real_spawn = _mp.mp.spawn
    calls = {"n": 0}

    def flaky_spawn(*a, **kw):
        calls["n"] += 1
        if calls["n"] == 1:
            raise RuntimeError("The server socket has failed to listen ... EADDRINUSE, address already in use")
        return real_spawn(*a, **kw)

    monkeypatch.setattr(_mp.mp, "spawn", flaky_spawn)
    monkeypatch.setattr(_mp.time, "sleep", lambda s: None)
    assert _mp.run_ranks(_healthy, 2, "gloo") == [3.0, 3.0]
    assert calls["n"] == 2

    def broken_spawn(*a, **kw):
        calls["n"] += 1
        raise RuntimeError("something else")

    monkeypatch.setattr(_mp.mp, "spawn", broken_spawn)
    with pytest.raises(AssertionError, match="something else"):
        _mp.run_ranks(_healthy, 2, "gloo")
    assert calls["n"] == 3
