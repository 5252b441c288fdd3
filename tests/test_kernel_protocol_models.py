"""CPU restatements of two pieces of in-kernel logic, checked against their specifications.

1. The hand-over of epilogue chunk buffers between the epilogue warps and the push warp of the
   fused kernels (csrc/gemm/fo_gemm_sm100.cuh): EPI buffers, one `ready` and one `free` mbarrier per
   buffer, phase parities derived from a running chunk count, and - for EPI > 2 - buffers handed
   back EPI - 1 chunks after their stores were issued (`cp.async.bulk.wait_group.read EPI-1`).
   The model runs both sides under random interleavings and checks that no buffer is refilled
   while a store may still read it, that every chunk is pushed exactly once and in order, and
   that neither side gets stuck.
2. The arithmetic of the RMSNorm tail of the reduce-scatter reducers: sum the partials in fp32,
   round, accumulate the squares of the ROUNDED values, then y = round(round(x * scale) * w).
"""
import random

import pytest
import torch

from flashoverlap_b200.utils import layout


class _Mbar:
    """mbarrier with an arrival count; wait(parity) passes when the phase with that parity is complete."""

    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase + 1

    def passed(self, parity):
        # the phase with parity `parity` is complete iff the current (incomplete) phase has the other parity
        return (self.phase & 1) != parity


@pytest.mark.parametrize("epi", [2, 3, 4])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_chunk_buffer_handover(epi, seed):
    rng = random.Random(seed * 10 + epi)
    n_chunks = 57
    ready = [_Mbar(1) for _ in range(epi)]     # one arrival stands for the 128 epilogue threads
    free = [_Mbar(1) for _ in range(epi)]
    owner = [None] * epi                       # chunk currently held by each buffer
    reading = [False] * epi                    # a store may still read the buffer
    pushed = []
    committed = []                             # chunks whose stores were issued, oldest first; reads finish in order
    reads_done = 0
    e_chunk, p_chunk = 0, 0
    steps = 0
    while (e_chunk < n_chunks or p_chunk < n_chunks) and steps < 100000:
        steps += 1
        who = rng.choice("eepr")
        if who == "e" and e_chunk < n_chunks:
            b = e_chunk % epi
            if free[b].passed(((e_chunk // epi) & 1) ^ 1):
                assert not reading[b], f"buffer {b} refilled while chunk {owner[b]} may still be read"
                owner[b] = e_chunk
                ready[b].arrive()
                e_chunk += 1
        elif who == "p" and p_chunk < n_chunks:
            b = p_chunk % epi
            if not ready[b].passed((p_chunk // epi) & 1):
                continue
            # issue + commit the stores of this chunk
            assert owner[b] == p_chunk
            reading[b] = True
            committed.append(p_chunk)
            pushed.append(p_chunk)
            # wait_group.read N: at most N of the newest groups may still be reading
            allowed = 0 if epi == 2 else epi - 1
            while len(committed) - reads_done > allowed:
                reading[committed[reads_done] % epi] = False
                reads_done += 1
            if epi == 2:
                free[b].arrive()
            elif p_chunk >= epi - 1:
                free[(p_chunk - (epi - 1)) % epi].arrive()
            p_chunk += 1
        elif who == "r" and reads_done < len(committed):
            reading[committed[reads_done] % epi] = False      # the hardware finishes reads on its own schedule
            reads_done += 1
    assert pushed == list(range(n_chunks)), "a side got stuck or chunks were reordered"


@pytest.mark.parametrize("ws", [2, 4, 8])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_rmsnorm_tail_arithmetic(ws, dt):
    torch.manual_seed(ws)
    rows, N, BN, eps = 16, 1024, 256, 1e-5
    partial = (torch.randn(ws, rows, N) * 0.5).to(dt)             # what the ranks pushed
    w = (1 + 0.1 * torch.randn(N)).to(dt)
    # reducers, tile by tile: fp32 sum, round, squares of the rounded values per row
    shard = torch.empty(rows, N, dtype=dt)
    ssq = torch.zeros(rows, dtype=torch.float32)
    for tn in range(N // BN):
        cols = slice(tn * BN, (tn + 1) * BN)
        s = partial[:, :, cols].float().sum(0).to(dt)
        shard[:, cols] = s
        ssq += s.float().pow(2).sum(-1)
    # the CTA that reduced the panel's last tile normalises it in place
    scale = torch.rsqrt(ssq / N + eps)
    y = (shard.float() * scale[:, None]).to(dt) * w
    want = layout.rmsnorm_ref(partial.float().sum(0).to(dt), w, eps)
    # identical up to the order in which the fp32 squares are added
    assert (y.float() - want.float()).abs().max().item() <= 2 * torch.finfo(dt).eps * want.float().abs().max().item()
