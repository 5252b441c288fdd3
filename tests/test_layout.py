"""Layout oracle: tile orders, reordered layout, reduce-scatter row maps (CPU)."""

import pytest
import torch

from flashoverlap_b200.utils import layout


def test_reorder_indices_matches_definition():
    hint = [5, 2, 7, 0]
    ra = layout.reorder_indices(8, hint).tolist()
    # hinted tiles take positions 0.., the rest follow in ascending id order
    assert [ra[h] for h in hint] == [0, 1, 2, 3]
    rest = [t for t in range(8) if t not in hint]
    assert [ra[t] for t in rest] == [4, 5, 6, 7]
    assert sorted(ra) == list(range(8))


def test_reorder_indices_rejects_bad_hint():
    with pytest.raises(ValueError):
        layout.reorder_indices(4, [0, 0])
    with pytest.raises(ValueError):
        layout.reorder_indices(4, [4])


@pytest.mark.parametrize("tm,tn,strip", [(4, 8, 8), (4, 8, 3), (5, 7, 2), (3, 4, 1), (2, 5, 0), (6, 6, 16)])
def test_raster_order_is_strip_major_permutation(tm, tn, strip):
    order = layout.raster_order(tm, tn, strip)
    assert sorted(order) == list(range(tm * tn))
    s = strip if 0 < strip <= tn else tn
    # first strip: M-major over the first s columns
    first = [m * tn + j for m in range(tm) for j in range(min(s, tn))]
    assert order[: len(first)] == first


def test_raster_order_units():
    # units of 4 vertically adjacent tiles (CTA pairs with two halves each), strips 2 tiles wide
    order = layout.raster_order(8, 4, 2, rows_per_unit=4)
    assert sorted(order) == list(range(32))
    assert order[:8] == [0, 4, 8, 12, 1, 5, 9, 13] and order[8:12] == [16, 20, 24, 28]
    assert layout.raster_order(4, 2, 2, True) == [0, 2, 1, 3, 4, 6, 5, 7]
    with pytest.raises(ValueError):
        layout.raster_order(6, 4, 2, rows_per_unit=4)


@pytest.mark.parametrize("rldn", [1, 2])
def test_reordered_roundtrip_and_addressing(rldn):
    torch.manual_seed(0)
    M, N, BM, BN = 512, 1024, 128, 256
    tiles = (M // BM) * (N // BN)
    RA = torch.randperm(tiles, dtype=torch.int32)
    C = torch.randn(M, N)
    buf = layout.to_reordered(C, BM, BN, RA, rldn)
    assert torch.equal(layout.from_reordered(buf, M, N, BM, BN, RA, rldn), C)
    # spot-check the closed-form address: C[i,j] lives at
    # ((r//L)*BM + i%BM) * (L*BN) + (r%L)*BN + j%BN with r = RA[tile]
    for i, j in [(0, 0), (130, 300), (511, 1023), (257, 512)]:
        r = int(RA[(i // BM) * (N // BN) + j // BN])
        off = ((r // rldn) * BM + i % BM) * (rldn * BN) + (r % rldn) * BN + j % BN
        assert buf[off] == C[i, j]


def test_row_mapping_gives_strided_ownership():
    """After the RE scatter, a plain reduce-scatter of each group's range hands rank p the
    logical rows i with i % ws == p, as tiles of BM/ws rows in reordered tile order."""
    torch.manual_seed(1)
    M, N, BM, BN, ws = 512, 512, 128, 256, 4
    tm, tn = M // BM, N // BN
    hint = layout.raster_order(tm, tn, 1)
    RA = layout.reorder_indices(tm * tn, hint)
    cseg = [3, 5]
    RE = layout.generate_row_mapping(M, N, BM, BN, cseg, ws).long()
    assert sorted(RE.tolist()) == list(range(M * N // BN))
    C = torch.randn(M, N)
    rows = layout.to_reordered(C, BM, BN, RA).reshape(-1, BN)
    scattered = torch.empty_like(rows)
    scattered[RE] = rows
    flat = scattered.reshape(-1)
    for p in range(ws):
        parts = []
        for start, length in layout.group_ranges(cseg, BM * BN):
            seg = flat[start:start + length]
            parts.append(seg.reshape(ws, -1)[p])       # what reduce-scatter gives rank p
        shard = torch.cat(parts)
        got = layout.from_reordered(shard, M // ws, N, BM // ws, BN, RA)
        assert torch.equal(got, C[p::ws])
        assert torch.equal(got, layout.reorder_rows_by_world_size(C, ws)[p * (M // ws):(p + 1) * (M // ws)])
        assert torch.equal(layout.owned_rows(M, BM, ws, p, strided=True), torch.arange(M)[p::ws])


def test_owned_rows_contiguous_blocks():
    rows = layout.owned_rows(256, 128, 4, 1, strided=False)
    assert rows.tolist() == list(range(32, 64)) + list(range(160, 192))


def test_wave_groups_and_compositions():
    assert layout.waves_of(300, 146) == [146, 146, 8]
    assert layout.cseg_from_wave_groups(300, 146, [1, 2]) == [146, 154]
    with pytest.raises(ValueError):
        layout.cseg_from_wave_groups(300, 146, [1, 1])
    comps = list(layout.integer_compositions(4))
    assert len(comps) == 8 and all(sum(c) == 4 for c in comps)
    assert len({tuple(c) for c in comps}) == 8
    assert list(layout.integer_compositions(3, max_parts=1)) == [[3]]


def test_rmsnorm_ref_matches_manual():
    x = torch.randn(4, 64)
    w = torch.rand(64) + 0.5
    y = layout.rmsnorm_ref(x, w, 1e-6)
    manual = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w
    assert torch.allclose(y, manual, atol=1e-6)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gathered_views_restore_token_order(world):
    """Shards cut by the contiguous-block ownership, concatenated in rank order (what an
    all-gather delivers), read through gathered_as_tokens are the tokens in order; an
    elementwise op over rank-major inputs with tokens_as_gathered(out) as its destination
    lands in token order."""
    T, c, BM = 512, 24, 128
    tokens = torch.arange(T * c, dtype=torch.float32).reshape(T, c)
    shards = [tokens[layout.owned_rows(T, BM, world, r, strided=False)] for r in range(world)]
    gathered = torch.cat(shards)
    assert torch.equal(layout.gathered_as_tokens(gathered, world, BM).reshape(T, c), tokens)
    # column slices of a wider rank-major matrix, as the gate / up halves of an MLP are
    wide = torch.cat([gathered, 2 * gathered], dim=1)
    a, b = wide.split([c, c], dim=1)
    n, ro = T // world, BM // world
    out = torch.full((T, c), float("nan"))
    torch.mul(a.reshape(world, n // ro, ro, c), b.view(world, n // ro, ro, c),
              out=layout.tokens_as_gathered(out, world, BM))
    assert torch.equal(out, 2 * tokens * tokens)
