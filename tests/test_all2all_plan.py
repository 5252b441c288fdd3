"""Row bookkeeping of the fused GEMM+all-to-all, checked on the CPU against the oracle."""
import numpy as np
import pytest
import torch

from flashoverlap_b200.utils import layout


def _plan(lib, mlen, rank):
    flat = list(torch.ops.flashoverlap_op.all2all_plan(mlen, rank))
    return flat[:8], flat[8:16], flat[16], flat[17]


@pytest.mark.parametrize("ws", [2, 4, 8])
def test_plan_matches_oracle(lib, ws):
    rng = np.random.default_rng(ws)
    mlen = torch.tensor(rng.integers(0, 200, size=(ws, ws)), dtype=torch.int32)
    N = 4
    C = []
    for r in range(ws):
        rows = int(mlen[r].sum() - mlen[r][r]) + 7          # a few rows past the last run
        C.append(torch.arange(rows * N, dtype=torch.float32).reshape(rows, N) + 1000.0 * r)
    want = layout.all2all_reference(C, mlen.tolist())
    got = [torch.full_like(w, float("nan")) for w in want]
    for r in range(ws):
        row_end, dst_row, send_rows, recv_rows = _plan(lib, mlen, r)
        assert send_rows == int(mlen[r].sum() - mlen[r][r])
        assert recv_rows == want[r].shape[0]
        # what the kernel's epilogue does for every row m of rank r's product
        for m in range(C[r].shape[0]):
            d, start = 0, 0
            while d < ws and m >= row_end[d]:
                start = row_end[d]
                d += 1
            if d == ws:
                assert m >= send_rows
                continue
            assert d != r
            got[d][dst_row[d] + m - start] = C[r][m]
    for g, w in zip(got, want):
        assert torch.equal(g, w)


def test_plan_rejects_bad_input(lib):
    with pytest.raises(RuntimeError):
        torch.ops.flashoverlap_op.all2all_plan(torch.zeros(2, 3, dtype=torch.int32), 0)
    with pytest.raises(RuntimeError):
        torch.ops.flashoverlap_op.all2all_plan(torch.zeros(2, 2, dtype=torch.int32), 2)
