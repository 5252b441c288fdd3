"""CPU restatements of pieces of in-kernel logic, checked against their specifications.

1. The hand-over of epilogue chunk buffers between the epilogue warps and the push warp of the
   fused kernels (csrc/gemm/fo_gemm_sm100.cuh): EPI buffers, one `ready` and one `free` mbarrier per
   buffer, phase parities derived from a running chunk count, and - for EPI > 2 - buffers handed
   back EPI - 1 chunks after their stores were issued (`cp.async.bulk.wait_group.read EPI-1`).
   The model runs both sides under random interleavings and checks that no buffer is refilled
   while a store may still read it, that every chunk is pushed exactly once and in order, and
   that neither side gets stuck.
2. The arithmetic of the RMSNorm tail of the reduce-scatter reducers: sum the partials in fp32,
   round, accumulate the squares of the ROUNDED values, then y = round(round(x * scale) * w).
3. The cross-rank protocol of the fused collectives over several back-to-back calls - arrival
   counters, `done` epochs, counter clearing by a rank's last CTA, staging reuse - for the push
   and the pull protocol, under random interleavings of all ranks' CTAs.
4. The `ready` / `done` handshakes that frame the fused GEMM + all-to-all.
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


class _RankState:
    def __init__(self, ws, ctas, tiles):
        self.flags = [0] * tiles                       # arrival counters of this rank (as owner)
        self.done = 0                                  # ranks that have completed a call, cumulative
        self.local_cnt = 0
        self.stage = [[None] * tiles for _ in range(ws)]   # [source rank][tile] -> call that wrote it
        self.call = 0                                  # call this rank's kernel is running (1-based), 0 = idle
        self.cta = []


@pytest.mark.parametrize("comm", ["all_reduce", "reduce_scatter"])
@pytest.mark.parametrize("pull", [False, True])
@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_cross_rank_counters_under_random_interleavings(comm, pull, seed):
    """Arrival counters, `done` epochs, flag clearing by the last CTA and staging reuse over
    several back-to-back calls, for the push protocol (partials stored into the owners' staging)
    and the pull protocol (partials kept in the producer's staging, owners read them): every
    reducer must find, for every tile, the partials of the CURRENT call from every rank, and
    nobody may get stuck."""
    rng = random.Random(seed)
    ws, ctas, tiles, calls = 3, 4, 10, 3
    ranks = [_RankState(ws, ctas, tiles) for _ in range(ws)]

    def start_call(r):
        st = ranks[r]
        st.call += 1
        my_tiles = lambda c: [t for t in range(tiles) if t % ctas == c]
        st.cta = [{"push": {"tiles": my_tiles(c), "i": 0, "started": False},
                   "red": {"tiles": my_tiles(c), "i": 0, "phase": "tiles"}} for c in range(ctas)]

    for r in range(ws):
        start_call(r)
    consumed = 0
    for _ in range(400000):
        if all(st.call == calls and all(c["red"]["phase"] == "exit" for c in st.cta) for st in ranks):
            break
        r = rng.randrange(ws)
        st = ranks[r]
        if all(c["red"]["phase"] == "exit" for c in st.cta):
            if st.call < calls:
                start_call(r)                           # next kernel on this rank's stream
            continue
        c = st.cta[rng.randrange(ctas)]
        epoch = st.call
        if rng.random() < 0.5:
            p = c["push"]
            if not p["started"]:
                if st.done >= ws * (epoch - 1):          # peers have consumed the previous call's staging
                    p["started"] = True
                continue
            if p["i"] < len(p["tiles"]):
                t = p["tiles"][p["i"]]
                for o in range(ws):                      # stores complete, then the arrival is announced
                    if pull:
                        ranks[r].stage[r][t] = epoch     # own staging only; the owners will read it
                    else:
                        ranks[o].stage[r][t] = epoch
                for o in range(ws):
                    ranks[o].flags[t] += 1
                p["i"] += 1
        else:
            q = c["red"]
            if q["phase"] == "tiles":
                if q["i"] == len(q["tiles"]):
                    st.local_cnt += 1
                    if st.local_cnt == ctas:             # last CTA of this rank
                        st.flags = [0] * tiles
                        st.local_cnt = 0
                        for o in range(ws):
                            ranks[o].done += 1
                        q["phase"] = "wait_done" if comm == "all_reduce" else "exit"
                    else:
                        q["phase"] = "exit"
                    continue
                t = q["tiles"][q["i"]]
                assert st.flags[t] <= ws, "an arrival of another call leaked into this one"
                if st.flags[t] == ws:
                    seen = [ranks[s].stage[s][t] if pull else st.stage[s][t] for s in range(ws)]
                    assert all(v == epoch for v in seen), f"rank {r} tile {t}: staging holds calls {seen} in call {epoch}"
                    consumed += 1
                    q["i"] += 1
            elif q["phase"] == "wait_done":
                if st.done >= ws * epoch:
                    q["phase"] = "exit"
    else:
        raise AssertionError("the protocol got stuck")
    assert consumed == ws * tiles * calls


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_all2all_handshakes_under_random_interleavings(seed):
    """Fused GEMM + all-to-all: `ready` counters (a receive buffer is written only after its owner
    has entered the call, i.e. after its reader of the previous call) and `done` counters (the
    kernel ends only when every rank has sent everything).  The reader that follows each kernel
    on a rank's stream must see the rows of exactly that call from every peer."""
    rng = random.Random(seed)
    ws, ctas, calls = 3, 3, 4
    recv = [[0] * ws for _ in range(ws)]        # recv[o][s]: call whose rows from s sit in o's buffer
    ready = [0] * ws
    done = [0] * ws
    local_cnt = [0] * ws
    state = [{"call": 0, "phase": "idle", "cta": []} for _ in range(ws)]

    def start(r):
        st = state[r]
        st["call"] += 1
        st["phase"] = "kernel"
        st["cta"] = [{"step": "announce" if c == 0 else "wait_ready"} for c in range(ctas)]

    for r in range(ws):
        start(r)
    reads = 0
    for _ in range(200000):
        if all(st["call"] == calls and st["phase"] == "finished" for st in state):
            break
        r = rng.randrange(ws)
        st = state[r]
        k = st["call"]
        if st["phase"] == "read":                       # the consumer of this call's rows
            for s in range(ws):
                if s != r:
                    assert recv[r][s] == k, f"rank {r} reads rows of call {recv[r][s]} from {s} in call {k}"
            reads += 1
            st["phase"] = "finished" if k == calls else "idle"
            if st["phase"] == "idle":
                start(r)
            continue
        if st["phase"] != "kernel":
            continue
        c = st["cta"][rng.randrange(ctas)]
        if c["step"] == "announce":
            for o in range(ws):
                ready[o] += 1
            c["step"] = "wait_ready"
        elif c["step"] == "wait_ready":
            if ready[r] >= ws * k:
                c["step"] = "store"
        elif c["step"] == "store":
            for o in range(ws):
                if o != r:
                    assert state[o]["call"] == k and state[o]["phase"] == "kernel", \
                        f"rank {r} writes call {k} into rank {o} which is in call {state[o]['call']} ({state[o]['phase']})"
                    recv[o][r] = k
            local_cnt[r] += 1
            if local_cnt[r] == ctas:
                local_cnt[r] = 0
                for o in range(ws):
                    done[o] += 1
                c["step"] = "wait_done"
            else:
                c["step"] = "exit"
        elif c["step"] == "wait_done":
            if done[r] >= ws * k:
                c["step"] = "exit"
        if all(x["step"] == "exit" for x in st["cta"]):
            st["phase"] = "read"
    else:
        raise AssertionError("the handshake got stuck")
    assert reads == ws * calls


@pytest.mark.parametrize("ring", [1, 4, 8])
@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_signal_ring_between_push_and_signal_warp(ring, seed):
    """The ring through which the push warp hands finished tiles to the signal warp of the fused
    kernels (csrc/gemm/fo_gemm_sm100.cuh: sig_full / sig_empty mbarriers, slot = count % ring,
    parities from the running counts; the signal warp takes every slot that is already full and
    publishes the batch behind ONE fence).  Under random interleavings: a slot is never rewritten
    before the signal warp has read it, every tile is published exactly once and in order, a tile
    is never published before its stores completed, and both sides terminate."""
    rng = random.Random(100 * ring + seed)
    n_tiles = 41
    full = [_Mbar(1) for _ in range(ring)]
    empty = [_Mbar(1) for _ in range(ring)]
    slot_tile = [None] * ring
    slot_unread = [False] * ring
    stores_done = set()
    published = []
    fences = 0
    handed, taken = 0, 0
    steps = 0
    while taken < n_tiles and steps < 200000:
        steps += 1
        if rng.random() < 0.5:
            if handed < n_tiles:
                s = handed % ring
                if not empty[s].passed(((handed // ring) & 1) ^ 1):
                    continue                      # ring full: the push warp waits (bounded in the kernel)
                stores_done.add(handed)           # cp.async.bulk.wait_group: the tile's stores have landed
                assert not slot_unread[s], f"slot {s} rewritten before tile {slot_tile[s]} was read"
                slot_tile[s], slot_unread[s] = handed, True
                full[s].arrive()
                handed += 1
        else:
            s = taken % ring
            if not full[s].passed((taken // ring) & 1):
                continue
            m = 1
            while taken + m < n_tiles and m < ring and full[(taken + m) % ring].passed(((taken + m) // ring) & 1):
                m += 1
            fences += 1                           # one system-scope release fence for the whole batch
            for j in range(m):
                sj = (taken + j) % ring
                t = slot_tile[sj]
                assert t == taken + j and t in stores_done
                published.append(t)
                slot_unread[sj] = False
                empty[sj].arrive()
            taken += m
    assert published == list(range(n_tiles))
    assert fences <= n_tiles and (ring == 1 or fences >= 1)
