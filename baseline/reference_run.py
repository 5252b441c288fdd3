"""Runs the unmodified reference library for bench.py's reference arm.

Only the reference's own objects are used on the measured paths:
``torch.classes.flashoverlap_class.{OverlapImpl,BaselineImpl}`` and
``torch.ops.flashoverlap_op.reorder_rmsnorm`` from ``baseline/_ref/lib/libst_pybinding.so``
(built by CMake from an untouched copy of the reference sources, CUTLASS headers taken from the
``flashinfer`` wheel) and ``reorder_indices`` / ``generate_row_mapping`` from its
``example/utils.py``.  This module never imports this repository's package or native library.

What is timed (all fp16 - the reference has no other type - with fp16 accumulation):
  * headline: GEMM+AllReduce of the benchmark shape through ``gemm_allreduce_overlap``
    (src/overlap_impl.cu:214-264), tuned as below;
  * ``baseline_impl_ms``: the reference's own non-overlap baseline for the same shape,
    ``BaselineImpl.gemm_allreduce`` = cuBLAS fp16 + ncclAllReduce (src/baseline_impl.cu:28-63);
  * ``rs_rmsnorm_ms``: GEMM+ReduceScatter+RMSNorm of the sequence-parallel shape through
    ``gemm_reducescatter_overlap`` + ``reorder_rmsnorm`` (src/overlap_impl.cu:266-321,
    src/rmsnorm/rmsnorm.cu:14-30), driven as in example/correctness_rs.py:21-71;
  * ``rs_baseline_impl_ms``: ``BaselineImpl.gemm_reducescatter`` (src/baseline_impl.cu:65-108)
    followed by the RMSNorm of its example module (example/RMSNorm.py:7-18, torch ops).

Tuning inputs are produced in-process the way the reference's scripts produce them:
  1. Algo: every instantiation is timed through ``cutlass_gemm`` and the fastest are kept
     (tune/profile_config.py:85-93);
  2. hint: monitor-mode runs with the identity tile order; tiles whose completion rank falls into
     the same wave in all 10 samples form that wave; a candidate whose waves are not stable is
     rejected (tune/search.py:111-157); rank 0's hint is used by every rank (:178); when no
     candidate is stable (its tuner then stops with "Tuning fails", :414) the tile order of one
     monitor run is used instead - any permutation is a correct hint, only less well matched;
  3. cSeg: a handful of wave partitions (all-in-one = its non-overlapped path, halves, thirds,
     quarters, one wave per group) are timed and the fastest kept - a subset of its exhaustive
     search (tune/search.py:387-439), whose full 2**(waves-1) enumeration does not fit a benchmark.
"""
from __future__ import annotations

import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def last_run_path(world: int) -> str:
    """Where the arm leaves its JSON line for the product arm's ratio columns (git-ignored)."""
    return os.path.join(REF_DIR, f"last_run_tp{world}.json")


class _Case:
    """One shape and collective driven through the reference's OverlapImpl."""

    def __init__(self, torch, dist, ref, impl, kind, M, N, K, dev, rank, world, sm_count, algo_params):
        self.torch, self.dist, self.ref, self.impl = torch, dist, ref, impl
        self.kind, self.M, self.N, self.K = kind, M, N, K            # kind: "ar" | "rs"
        self.dev, self.rank, self.world, self.sm_count = dev, rank, world, sm_count
        self.algo_params = algo_params
        self.A = (torch.randn(M, K, device=dev) * 0.02).to(torch.float16)
        self.B = (torch.randn(N, K, device=dev) * 0.02).to(torch.float16)
        self.C = torch.empty(M, N, device=dev, dtype=torch.float16)
        if kind == "rs":
            self.D = torch.empty(M // world, N, device=dev, dtype=torch.float16)
            self.Y = torch.empty_like(self.D)
            self.w = (1 + 0.02 * torch.randn(N, device=dev)).to(torch.float16)

    # ---- the reference's calls
    def overlap(self, a, mm, RA, RE, cc, cg, algo, monitor):
        if self.kind == "ar":
            self.impl.gemm_allreduce_overlap(a, self.B, self.C, mm, RA, 1, cc, cg, algo, monitor)
        else:
            self.impl.gemm_reducescatter_overlap(a, self.B, self.C, self.D, mm, RA, RE, 1, cc, cg, algo, monitor)

    def nonoverlap(self, a, algo):
        if self.world == 1:
            # With one rank nccl_init leaves the communicator null (src/overlap_impl.cu:56-59) and the
            # collective calls would pass it to NCCL and exit; a collective over one rank is the
            # identity, so the comparable stock call is the GEMM alone.
            self.impl.cutlass_gemm(a, self.B, self.C, algo)
        elif self.kind == "ar":
            self.impl.gemm_allreduce(a, self.B, self.C, algo)
        else:
            self.impl.gemm_reducescatter(a, self.B, self.C, self.D, algo)

    def norm_reordered(self, BM, BN, RA):
        self.torch.ops.flashoverlap_op.reorder_rmsnorm(self.D, self.Y, self.w, BM // self.world, BN, 1, RA)

    def norm_plain(self, x):
        # the RMSNorm module of its examples (example/RMSNorm.py:7-18), eps 1e-5
        t = self.torch
        xf = x.float()
        return (xf * t.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).type_as(x) * self.w

    def row_mapping(self, BM, BN, cseg):
        return self.ref["generate_row_mapping"](self.M, self.N, BM, BN, cseg, self.world) if self.kind == "rs" \
            else self.torch.zeros(1, dtype=self.torch.int32, device=self.dev)


def _t_of(torch, fn, reps=3, warm=1):
    for _ in range(warm):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(reps):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps


def _tune(case: _Case):
    """Returns (step(a=None), path description, tuning record) for the case."""
    torch, dist, ref = case.torch, case.dist, case.ref
    impl, dev, rank, world = case.impl, case.dev, case.rank, case.world
    M, N = case.M, case.N
    div_up, reorder_indices = ref["div_up"], ref["reorder_indices"]

    def agree(values):
        t = torch.tensor(values, device=dev, dtype=torch.float32)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    # 1. Algo
    n_algos = len(case.algo_params)
    gemm_ms = agree([_t_of(torch, lambda a=a: impl.cutlass_gemm(case.A, case.B, case.C, a)) for a in range(n_algos)])
    ranked = sorted(range(n_algos), key=lambda a: gemm_ms[a])[:5]
    tuning = {"gemm_ms_best5": {int(a): round(gemm_ms[a], 4) for a in ranked}}
    name = "gemm_allreduce" if case.kind == "ar" else "gemm_reducescatter"

    def finish_nonoverlap(algo, why):
        def step(a=None):
            case.nonoverlap(case.A if a is None else a, algo)
            if case.kind == "rs":
                case.Y = case.norm_plain(case.C if world == 1 else case.D)
        tuning["Algo"] = int(algo)
        call = "cutlass_gemm" if world == 1 else name
        tail = " + RMSNorm (torch ops of its example module)" if case.kind == "rs" else ""
        return step, f"OverlapImpl.{call}{tail} ({why})", tuning

    if world == 1:
        return finish_nonoverlap(ranked[0], "one rank: no communicator, the collective is the identity")

    # 2. hint by monitor runs
    chosen, one_run = None, None
    # wave window: one wave of (SMs - 2) tiles as in its exhaustive search, then the coarser
    # window of its predictive search (ceil(waves / 10) waves, tune/search.py:462-466)
    for coarse in (False, True):
        for algo in ranked:
            BM, BN = case.algo_params[algo][0], case.algo_params[algo][1]
            tm, tn = div_up(M, BM), div_up(N, BN)
            tiles = tm * tn
            base_w = case.sm_count - 2
            wsize = base_w * (div_up(div_up(tiles, base_w), 10) if coarse else 1)
            waves = div_up(tiles, wsize)
            cseg = [min(wsize, tiles - i * wsize) for i in range(waves)]
            cseg_cpu = torch.tensor(cseg, dtype=torch.int32)
            cseg_gpu = cseg_cpu.to(dev)
            mm = torch.zeros(tm + 1, tn, dtype=torch.int32, device=dev)
            ident = torch.arange(tiles, dtype=torch.int32, device=dev).reshape(tm, tn)
            RE = case.row_mapping(BM, BN, cseg)
            for _ in range(10):
                case.overlap(case.A, mm, ident, RE, cseg_cpu, cseg_gpu, algo, True)
            samples = torch.empty(10, tiles, dtype=torch.int32, device=dev)
            for i in range(10):
                mm[0] = 0
                case.overlap(case.A, mm, ident, RE, cseg_cpu, cseg_gpu, algo, True)
                samples[i] = mm[1:].reshape(-1)
            torch.cuda.synchronize()
            if one_run is None:
                one_run = (algo, BM, BN, tm, tn, tiles, wsize, waves, samples[-1].clone())
            hint, ok = [], True
            for w in range(waves):
                idx = torch.where(((samples >= w * wsize) & (samples < (w + 1) * wsize)).sum(0) == 10)[0]
                if w < waves - 1 and idx.numel() < wsize:
                    ok = False
                    break
                hint += idx.tolist()
            flag = torch.tensor([1.0 if ok else 0.0], device=dev)
            dist.broadcast(flag, src=0)           # every rank follows rank 0's verdict and hint
            if flag.item() < 0.5:
                continue
            payload = [hint if rank == 0 else None]
            dist.broadcast_object_list(payload, src=0)
            chosen = (algo, BM, BN, tm, tn, tiles, wsize, waves, payload[0])
            break
        if chosen is not None:
            break
    if chosen is None and one_run is not None:
        # Its tuner gives up here ("Tuning fails", tune/search.py:414).  To still give its overlap
        # path a chance, take the tile order of ONE monitor run of its fastest GEMM as the hint:
        # any permutation is a correct hint (groups are counted by membership, not by time), it
        # is only less well matched to the real completion order.  The wave groupings below
        # include its non-overlapped call, so the arm never gets slower by this.
        try:
            algo, BM, BN, tm, tn, tiles, wsize, waves, order = one_run
            payload = [torch.argsort(order.long()).tolist() if rank == 0 else None]
            dist.broadcast_object_list(payload, src=0)
            if sorted(payload[0]) == list(range(tiles)):
                chosen = (algo, BM, BN, tm, tn, tiles, wsize, waves, payload[0])
                tuning["hint"] = "order of one monitor run (its stability check failed)"
        except Exception as ex:
            tuning["hint_error"] = repr(ex)[:200]
            chosen = None
    if chosen is None:
        # No overlap config exists for this shape on this GPU.  What a user of the reference is
        # left with is its non-overlapped call, which is also what its speed test runs for a
        # single group (test/test.py:104-134).
        tuning["hint"] = "unstable"
        return finish_nonoverlap(ranked[0], "its tuner found no stable tile order: no overlap config")

    # 3. wave partition by timing
    try:
        algo, BM, BN, tm, tn, tiles, wsize, waves, hint = chosen
        RA = reorder_indices(tiles, hint).reshape(tm, tn)
        mm = torch.zeros(1, tn, dtype=torch.int32, device=dev)

        def partition(parts):
            base, rem = divmod(waves, parts)
            groups = [base + (1 if i < rem else 0) for i in range(parts)]
            out, acc = [], 0
            for j, g in enumerate(groups):
                n = g * wsize if j < parts - 1 else tiles - acc
                out.append(n)
                acc += n
            return out

        def overlap_step(cs):
            cc = torch.tensor(cs, dtype=torch.int32)
            cg = cc.to(dev)
            RE = case.row_mapping(BM, BN, cs)

            def step(a=None):
                case.overlap(case.A if a is None else a, mm, RA, RE, cc, cg, algo, False)
                if case.kind == "rs":
                    case.norm_reordered(BM, BN, RA)
            return step

        non_step, non_path, _ = finish_nonoverlap(algo, "its tuner found no overlap grouping faster")
        cands = [[tiles]] + [partition(p) for p in (2, 3, 4, 6) if p <= waves] + [partition(waves)]
        best = None
        for cs in cands:
            fn = non_step if len(cs) == 1 else overlap_step(cs)   # one group = its non-overlapped path (test/test.py:104-134)
            t = agree([_t_of(torch, fn, reps=10, warm=3)])[0]
            if best is None or t < best[0]:
                best = (t, cs, fn)
        t, cs, fn = best
        tuning.update(Algo=int(algo), BM=BM, BN=BN, cSeg=cs, probe_ms=round(t, 4))
        if len(cs) == 1:
            return non_step, non_path, tuning
        path = "OverlapImpl.gemm_allreduce_overlap" if case.kind == "ar" else \
            "OverlapImpl.gemm_reducescatter_overlap + flashoverlap_op.reorder_rmsnorm"
        if "hint" in tuning:
            path += " (hint: " + tuning["hint"] + ")"
        return fn, path, tuning
    except Exception as ex:  # its overlap path could not be set up: its non-overlapped call remains
        tuning["overlap_error"] = repr(ex)[:200]
        return finish_nonoverlap(chosen[0], "setting up its overlap path raised an exception")


def run(args, lib_path: str) -> None:
    import torch
    import torch.distributed as dist

    import bench

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29512")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    torch.ops.load_library(lib_path)
    sys.path.insert(0, os.path.join(REF_DIR, "example"))
    from utils import div_up, generate_row_mapping, reorder_indices  # the reference's own helpers
    ref = {"div_up": div_up, "generate_row_mapping": generate_row_mapping, "reorder_indices": reorder_indices}

    algo_dict = torch.load(os.path.join(REF_DIR, "configs", "AlgoDict.pt"))
    algo_params = {v: k for k, v in algo_dict.items()}
    sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
    flush = bench.make_flusher(torch)

    def nccl_id():
        if world == 1:
            return [0] * 16
        payload = [list(torch.ops.flashoverlap_op.generate_nccl_id()) if rank == 0 else None]
        dist.broadcast_object_list(payload, src=0)
        return payload[0]

    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.nccl_init(rank, world, nccl_id())
    impl.cutlass_init()
    impl.overlap_init()

    torch.manual_seed(1234 + rank)
    M, N, K = bench.M_AR, bench.N_AR, bench.K_AR_TOTAL // world
    case = _Case(torch, dist, ref, impl, "ar", M, N, K, dev, rank, world, sm_count, algo_params)
    step, path, tuning = _tune(case)
    A, C = case.A, case.C

    sampler = bench.ClockSampler(local) if rank == 0 else None
    ms, clocks, wall, blocks = bench.time_blocks(torch, dist, world, step, args.steps, args.warmup, flush, sampler)
    flops = 2.0 * M * N * bench.K_AR_TOTAL
    host_in = torch.empty(M, K, dtype=torch.float16).pin_memory()
    host_in.copy_(A)
    host_out = torch.empty(128, N, dtype=torch.float16).pin_memory()
    dev_bufs = [torch.empty_like(A), torch.empty_like(A)]
    e2e_steps = max(3, min(args.steps, 30))

    def step_on(a):
        step(a)
        return C

    e2e_ms = bench.e2e_pipeline(torch, dist, world, host_in, dev_bufs, step_on,
                                lambda out: out.view(-1)[: 128 * N].view(128, N), host_out, e2e_steps,
                                max(3, min(args.warmup, 5)))
    del host_in, dev_bufs

    # ---- the reference's other paths on the named shapes (extra columns, never the headline)
    extra = {"path": path, "note": "reference is fp16-only with fp16 accumulation (src/gemm/gemm.cu:33-49)",
             "ms_per_step_blocks": blocks}
    steps_x, warm_x = max(20, min(args.steps, 100)), 5
    if not getattr(args, "no_extra", False):
        try:
            base = torch.classes.flashoverlap_class.BaselineImpl()
            base.nccl_init(rank, world, nccl_id())
            base.cublas_init()
            # one rank: its gemm_allreduce returns before the GEMM when there is no communicator
            # (src/baseline_impl.cu:31-33), so the GEMM alone is timed
            fn = (lambda: base.cublas_gemm(A, case.B, C)) if world == 1 else (lambda: base.gemm_allreduce(A, case.B, C))
            t, _, _ = bench.time_steps(torch, dist, world, fn, steps_x, warm_x, flush)
            extra["baseline_impl_ms"] = round(t, 5)
            extra["baseline_impl_path"] = "BaselineImpl.cublas_gemm" if world == 1 else "BaselineImpl.gemm_allreduce"
        except Exception as ex:
            extra["baseline_impl_error"] = repr(ex)[:200]
        try:
            del case, A, C, step
            torch.cuda.empty_cache()
            M2, N2, K2 = bench.M_RS, bench.N_RS, bench.K_RS_TOTAL // world
            rs = _Case(torch, dist, ref, impl, "rs", M2, N2, K2, dev, rank, world, sm_count, algo_params)
            rs_step, rs_path, rs_tuning = _tune(rs)
            t, _, _ = bench.time_steps(torch, dist, world, rs_step, steps_x, warm_x, flush)
            extra.update(rs_rmsnorm_ms=round(t, 5), rs_rmsnorm_path=rs_path, rs_rmsnorm_tuning=rs_tuning,
                         rs_shape={"M": M2, "N": N2, "K_per_rank": K2})

            def rs_base():
                if world == 1:
                    base.cublas_gemm(rs.A, rs.B, rs.C)
                    rs.Y = rs.norm_plain(rs.C)
                else:
                    base.gemm_reducescatter(rs.A, rs.B, rs.C, rs.D)
                    rs.Y = rs.norm_plain(rs.D)
            t, _, _ = bench.time_steps(torch, dist, world, rs_base, steps_x, warm_x, flush)
            extra["rs_baseline_impl_ms"] = round(t, 5)
        except Exception as ex:
            extra["rs_error"] = repr(ex)[:200]

    line = {
        "metric": "gemm_allreduce_tflops", "value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
        "impl": "reference",
        "config": bench.config_dict(M, N, K, world),
        "clocks": clocks,
        "e2e": {"value": round(flops / (e2e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms, 5),
                "steps": e2e_steps, "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": 128 * N * 2},
        "tuning": tuning, "extra": extra, "wall_s_timed_region": round(wall, 3),
    }
    if rank == 0:
        print(json.dumps(line), file=bench.REAL_STDOUT, flush=True)
        try:
            with open(last_run_path(world), "w") as f:
                json.dump(line, f)
        except OSError:
            pass
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
