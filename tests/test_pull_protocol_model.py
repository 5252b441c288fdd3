"""Index arithmetic of the pull protocol of the fused kernels, restated on the CPU.

Every rank stages its partial tile in its own buffer as [tile][owner][rows owned][BN] (the
epilogue groups a tile's rows by owner, the push warp stores whole 128-row chunks); owner `me`
then sums, over the ranks, the slice that starts `tile_off` bytes into each staging buffer and
writes row q of the slice to tile row `q * ws + me` (strided ownership) or `me * rows_owned + q`
(contiguous).  The model follows csrc/gemm/fo_gemm_sm100.cuh step by step and must reproduce
a plain sum of the partials.
"""
import numpy as np
import pytest

BM = 128


def _stage_tile(partial_tile, ws, strided):
    """Epilogue + push: tile rows -> staging rows of the tile's [owner][q] block."""
    rows_owned = BM // ws
    staged = np.empty_like(partial_tile)
    for my_row in range(BM):
        o = my_row % ws if strided else my_row // rows_owned
        q = my_row // ws if strided else my_row % rows_owned
        staged[o * rows_owned + q] = partial_tile[my_row]
    return staged


@pytest.mark.parametrize("ws", [2, 4, 8])
@pytest.mark.parametrize("strided", [True, False])
@pytest.mark.parametrize("bn", [128, 256])
def test_pull_protocol_reproduces_the_sum(ws, strided, bn):
    rng = np.random.default_rng(ws * 10 + bn + int(strided))
    tiles_m, tiles_n = 2, 3
    M, N = tiles_m * BM, tiles_n * bn
    rows_owned = BM // ws
    partial = rng.standard_normal((ws, M, N)).astype(np.float32)
    # staging of every rank: [tiles * 128, BN] elements
    stage = np.zeros((ws, tiles_m * tiles_n * BM, bn), np.float32)
    for s in range(ws):
        for tm in range(tiles_m):
            for tn in range(tiles_n):
                t = tm * tiles_n + tn
                tile = partial[s, tm * BM:(tm + 1) * BM, tn * bn:(tn + 1) * bn]
                stage[s, t * BM:(t + 1) * BM] = _stage_tile(tile, ws, strided)
    out = np.full((M, N), np.nan, np.float32)
    flat = stage.reshape(ws, -1)
    vec_per_row = bn // 8
    for me in range(ws):
        for tm in range(tiles_m):
            for tn in range(tiles_n):
                t = tm * tiles_n + tn
                tile_off = (t * BM + me * rows_owned) * bn          # elements
                out_base = tm * BM * N + tn * bn
                for v in range(rows_owned * vec_per_row):
                    q, c8 = divmod(v, vec_per_row)
                    src = tile_off + v * 8                          # vector v = bytes [16 v, 16 v + 16)
                    assert src + 8 <= flat.shape[1]
                    y = flat[:, src:src + 8].sum(0)
                    lr = q * ws + me if strided else me * rows_owned + q
                    off = out_base + lr * N + c8 * 8
                    out.reshape(-1)[off:off + 8] = y
    np.testing.assert_allclose(out, partial.sum(0), rtol=1e-6, atol=1e-6)
