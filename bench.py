#!/usr/bin/env python
"""Headline benchmark: fused GEMM+AllReduce of a row-parallel down-projection.

Config (fixed total work, split over the GPUs = strong scaling): per-rank A[M=8192, K=28672/tp]
and B[N=8192, K/tp], bf16 ~N(0, 0.02), fp32 accumulate, all-reduced output [8192, 8192] bf16.
One step = one ``OverlapImpl.gemm_allreduce_overlap`` call (one hand-written sm_100a kernel
that computes the tiles and all-reduces them over NVLink peer memory).  The value is the
whole-job rate 2*M*N*K_total / step time in TFLOP/s.

    python bench.py --gpus 1 --steps 200 --warmup 10
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29555 bench.py --gpus 8

Rank 0 prints ONE JSON line.  ``--impl reference`` runs the unmodified reference library from
``baseline/_ref`` through its own ``OverlapImpl`` for the same shape (fp16: it has no bf16).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_AR, N_AR, K_AR_TOTAL = 8192, 8192, 28672
M_RS, N_RS, K_RS_TOTAL = 16384, 8192, 8192
# Every arm is warmed for this long before it is timed: within one process the same kernel was seen
# 7 % apart between an arm timed half a second after the first load and one timed seconds later,
# while the board's power management was still settling under the 1 kW cap.
WARM_SECONDS = 1.0
CHECK_ROWS_PER_PANEL = 8     # rows of every 128-row panel compared with the fp32 reference
TIMED_BLOCKS = 9             # blocks of `steps` steps; the median block is the reported one
NVLINK_GBS = 770.0           # measured peer-copy bandwidth per direction per GPU (B200, NVLink 5)
REAL_STDOUT = sys.stdout
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["source"] = "fallback"
    return d


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with nvidia-smi while timing."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        import torch
        self.uuid = None
        try:
            u = str(torch.cuda.get_device_properties(device_index).uuid)
            self.uuid = u if u.startswith("GPU-") else "GPU-" + u
        except Exception:
            pass
        self.index = device_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            sel = ["-i", self.uuid] if self.uuid else ["-i", str(self.index)]
            self.proc = subprocess.Popen(
                ["nvidia-smi", *sel, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); pw.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm), power_w_max=max(pw))
        return out


def pick_algo(torch, dist, world, run, candidates, flush, reps=10, settle_seconds=0.35, check=None):
    """Fastest candidate, agreed on by all ranks (max over ranks per candidate).

    Every candidate is ranked in the regime of the timed region - under ITS OWN sustained load.
    The board runs at its 1 kW cap in the timed region, and the kernels differ in the power they
    draw per FLOP (operand bytes per FLOP, mostly), so the clock each one sustains is part of its
    time: a kernel that wins a short burst after another kernel's warm-up can lose by 10 % once the
    power controller has settled on it.  So each candidate first runs alone for `settle_seconds`,
    then is timed with per-call events and the L2 flushed between calls."""
    times = []
    for a in candidates:
        try:
            run(a)
            torch.cuda.synchronize()
            if check is not None and not check():
                # a candidate whose device-side waits give up is dropped after ONE call instead of
                # running into its time limit on every timed iteration
                raise RuntimeError("device status not ok")
            t0 = time.perf_counter()
            run(a)
            flush()
            torch.cuda.synchronize()
            one = torch.tensor([max(time.perf_counter() - t0, 1e-5)], device="cuda")
            if world > 1:
                dist.all_reduce(one, op=dist.ReduceOp.MAX)       # same number of settling steps on every rank
            for _ in range(int(min(2000, settle_seconds / one.item()))):
                run(a)
                flush()
            n = max(reps, int(min(400, 0.15 / one.item())))
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            for s, e in ev:
                flush()
                s.record()
                run(a)
                e.record()
            torch.cuda.synchronize()
            times.append(sum(s.elapsed_time(e) for s, e in ev) / n)
        except Exception:
            times.append(1e9)
    t = torch.tensor(times, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return candidates[int(t.argmin().item())], [round(x, 4) for x in t.tolist()]


def _settle(torch, dist, world, fn, warmup, flush):
    """Warm up by count AND by time: the GPU settles at its power-capped clocks only after a few
    hundred milliseconds of load, and every arm must be measured in that state.  The number of
    extra warm-up steps is agreed on by all ranks so that everybody runs the same sequence."""
    torch.cuda.synchronize()
    t_warm = time.perf_counter()
    for _ in range(warmup):
        fn()
        flush()
    torch.cuda.synchronize()
    per_step = torch.tensor([(time.perf_counter() - t_warm) / max(1, warmup)], device="cuda")
    if world > 1:
        dist.all_reduce(per_step, op=dist.ReduceOp.MAX)
    extra_warm = int(min(2000, max(0.0, WARM_SECONDS / max(per_step.item(), 1e-5) - warmup)))
    for _ in range(extra_warm):
        fn()
        flush()


def _timed_block(torch, dist, world, fn, steps, flush):
    """`steps` steps with per-step CUDA events on the launching stream, L2 flushed between steps
    (outside the event pairs), barrier + synchronize on both sides.  Returns (mean ms per step,
    max over ranks; wall seconds of the bracket)."""
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for s, e in ev:
        flush()
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = sum(s.elapsed_time(e) for s, e in ev) / steps
    t = torch.tensor([ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()), wall


def time_steps(torch, dist, world, fn, steps, warmup, flush, sampler=None):
    """One timed block after the warm-up.  Returns (ms per step, clock record, wall seconds)."""
    _settle(torch, dist, world, fn, warmup, flush)
    if sampler:
        sampler.start()
    ms, wall = _timed_block(torch, dist, world, fn, steps, flush)
    clocks = sampler.stop() if sampler else None
    return ms, clocks, wall


def time_blocks(torch, dist, world, fn, steps, warmup, flush, sampler=None, blocks=TIMED_BLOCKS):
    """The headline timing: after the warm-up, `blocks` back-to-back blocks of exactly `steps`
    steps, each bracketed by barrier + synchronize; the MEDIAN block is the reported one (a
    single block of tens of milliseconds moves by several per cent with the board's power
    management).  Returns (ms per step of the median block, clock record over all blocks, wall
    seconds of the median block, the sorted per-block values)."""
    _settle(torch, dist, world, fn, warmup, flush)
    if sampler:
        sampler.start()
    res = [_timed_block(torch, dist, world, fn, steps, flush) for _ in range(blocks)]
    clocks = sampler.stop() if sampler else None
    res.sort(key=lambda r: r[0])
    ms, wall = res[len(res) // 2]
    return ms, clocks, wall, [round(r[0], 5) for r in res]


def config_dict(M, N, K, world):
    """The benchmark configuration, identical for the product arm and the reference arm."""
    return {"model": "row-parallel down-proj GEMM+AllReduce (Llama-3-70B MLP shape)",
            "M": M, "N": N, "K_total": K_AR_TOTAL, "K_per_rank": K, "global_batch": M, "seq_len": None,
            "parallelism": f"tp{world}", "l2": "256 MB buffer written between timed steps"}


def e2e_pipeline(torch, dist, world, host_in, dev_bufs, step_on, result_slice, host_out, steps, warmup):
    """End-to-end loop through the public API: every step copies its input from pinned host
    memory, runs, and reads a slice of the result back.  The copy of step i+1 overlaps the
    compute of step i (two device input buffers, one copy stream)."""
    main = torch.cuda.current_stream()
    copy = torch.cuda.Stream()
    ready = [torch.cuda.Event() for _ in dev_bufs]
    free = [torch.cuda.Event() for _ in dev_bufs]

    def run(n):
        for i in range(n):
            b = i % len(dev_bufs)
            with torch.cuda.stream(copy):
                copy.wait_event(free[b])
                dev_bufs[b].copy_(host_in, non_blocking=True)
                ready[b].record(copy)
            main.wait_event(ready[b])
            out = step_on(dev_bufs[b])
            free[b].record(main)
            host_out.copy_(result_slice(out), non_blocking=True)

    for f in free:
        f.record(main)
    run(warmup)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(main)
    run(steps)
    e.record(main)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t = torch.tensor([s.elapsed_time(e) / steps], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def make_flusher(torch):
    buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")  # > 126 MB L2
    return lambda: buf.zero_()


def run_ours(args):
    import torch
    import torch.distributed as dist

    from flashoverlap_b200 import ops
    from flashoverlap_b200.parallel import bootstrap
    from flashoverlap_b200.utils import config, layout

    rank, world, local = bootstrap.init_distributed()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    dev = torch.device("cuda", local)
    peaks = load_peaks()
    torch.manual_seed(1234 + rank)
    flush = make_flusher(torch)
    impl = bootstrap.make_overlap_impl(rank, world)
    impl.set_option("timeout_ms", 3000)

    M, N, K = M_AR, N_AR, K_AR_TOTAL // world
    A = (torch.randn(M, K, device=dev) * 0.02).to(torch.bfloat16)
    B = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
    from flashoverlap_b200.parallel import symm
    C, uses_multicast = symm.alloc_allreduce_output(impl, (M, N), torch.bfloat16, multicast=not args.no_nvls)

    # Pull protocol of the fused kernel: partial tiles stay in this rank's staging buffer and the
    # owners fetch them, through the NVSwitch's in-switch reduction when the staging has a
    # multicast mapping.  Both protocols are candidates of the probe below.
    protocols = ["push"]
    stage_mc = False
    if world > 1 and args.protocol in ("auto", "pull"):
        try:
            _, stage_mc = symm.alloc_stage(impl, M, N, torch.bfloat16, multicast=not args.no_nvls)
            protocols = ["pull"] if args.protocol == "pull" else ["push", "pull"]
        except Exception:
            protocols = ["push"]

    def healthy():
        """True when no rank's device-side wait has given up; otherwise all ranks re-align their
        call counters (collective) and the caller drops whatever it was trying."""
        ok = torch.tensor([1 if impl.read_status()[0] == 0 else 0], device=dev, dtype=torch.int32)
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 1:
            return True
        impl.resync()
        return False

    state = {}

    def prepare(algo):
        if algo in state:
            return state[algo]
        cfg = config.default_solution(M, N, algo)
        tiles = (M // cfg["BM"]) * (N // cfg["BN"])
        RA = layout.reorder_indices(tiles, cfg["hint"], device=dev).reshape(M // cfg["BM"], N // cfg["BN"])
        mm = torch.zeros(1, max(N // cfg["BN"], 8), device=dev, dtype=torch.int32)
        state[algo] = (cfg, RA, mm)
        return state[algo]

    empty = torch.empty(0, dtype=torch.int32)
    empty_gpu = torch.empty(0, dtype=torch.int32, device=dev)

    def step_cand(cand, a=A):
        algo, proto = cand
        cfg, RA, mm = prepare(algo)
        if world > 1:
            impl.set_option("stage_local", 1 if proto == "pull" else 0)
        # per-tile flags (empty cSeg): the finest wave grouping, which the fused kernel prefers
        impl.gemm_allreduce_overlap(a, B, C, mm, RA, 1, empty, empty_gpu, algo, False)
        return C

    tuned = config.load_tuned(M, N, K, tp=world, comm_op="all_reduce", mode="fused", gpu="b200")
    if tuned is not None:
        cand, algo_times, cands = (int(tuned["Algo"]), tuned.get("protocol", protocols[-1])), None, None
        if cand[1] not in protocols:
            cand = (cand[0], protocols[-1])
    else:
        cands = [(a, pr) for pr in protocols for a in ((19, 3, 17, 1) if world <= 2 else (3, 1, 19, 17))]
        cand, algo_times = pick_algo(torch, dist, world, step_cand, cands, flush, check=healthy)
    algo, protocol = cand

    sampler = ClockSampler(local) if rank == 0 else None
    ms, clocks, wall, blocks = time_blocks(torch, dist, world, lambda: step_cand(cand), args.steps, args.warmup, flush, sampler)
    impl.check_status()
    flops = 2.0 * M * N * K_AR_TOTAL
    value = flops / (ms * 1e-3) / 1e12

    # correctness check of the timed path against torch: CHECK_ROWS_PER_PANEL rows out of every
    # 128-row panel, all columns, fp32 reference summed over the ranks
    cfg, RA, _ = prepare(algo)
    nat = ops.unreorder(C, M, N, cfg["BM"], cfg["BN"], RA)
    g = torch.Generator().manual_seed(7)
    rows = torch.cat([p * 128 + torch.randperm(128, generator=g)[:CHECK_ROWS_PER_PANEL] for p in range(M // 128)]).to(dev)
    ref = A[rows].float() @ B.float().t()
    if world > 1:
        dist.all_reduce(ref)
    check_err = float((nat[rows].float() - ref).abs().max().item())
    check_ref_max = float(ref.abs().max().item())
    del nat, ref

    # ---- end to end: pinned host input every step, result slice read back every step
    host_in = torch.empty(M, K, dtype=torch.bfloat16).pin_memory()
    host_in.copy_(A)
    host_out = torch.empty(128, N, dtype=torch.bfloat16).pin_memory()
    dev_bufs = [torch.empty_like(A), torch.empty_like(A)]
    e2e_steps = max(3, min(args.steps, 30))
    e2e_ms = e2e_pipeline(torch, dist, world, host_in, dev_bufs, lambda a: step_cand(cand, a),
                          lambda out: out.view(-1)[: 128 * N].view(128, N), host_out, e2e_steps,
                          max(3, min(args.warmup, 5)))
    impl.check_status()
    del host_in, dev_bufs

    # ---- roofline of the fused step
    S = M * N * 2
    t_gemm = 2.0 * M * N * K / (peaks["bf16_tflops"] * 1e12)
    t_link = (2.0 * S * (world - 1) / world) / (NVLINK_GBS * 1e9) if world > 1 else 0.0
    roof_ms = max(t_gemm, t_link) * 1e3

    how_reduced = "none (one rank)"
    if world > 1:
        how_reduced = ("pull: partials staged locally, owners sum them with multimem.ld_reduce (in-switch)" if stage_mc
                       else "pull: partials staged locally, owners sum them with peer loads") if protocol == "pull" \
            else "push: partials stored into the owners' staging with TMA, summed by the owners' reducer warps"
    extra = {"algo": algo, "protocol": protocol, "reduction": how_reduced,
             "probe_candidates": [list(c) for c in cands] if cands else None, "probe_ms": algo_times,
             "allreduce_broadcast": "multimem.st (NVLS)" if uses_multicast else "peer stores",
             "check_max_abs_err": check_err, "check_ref_max_abs": check_ref_max, "check_rows": int(rows.numel()),
             "ms_per_step_blocks": blocks,
             "timing": f"{TIMED_BLOCKS} blocks of `steps` steps (per-step CUDA events on the launching stream, mean over "
                       "the block, max over ranks); ms_per_step is the median block",
             "roofline_ms": round(roof_ms, 4), "roofline_frac": round(roof_ms / ms, 4),
             "roofline_peaks": peaks["source"], "wall_s_timed_region": round(wall, 3)}

    if not args.no_extra:
        try:
            extra.update(extras(torch, dist, impl, rank, world, dev, A, B, C, algo, flush, peaks, args.steps, protocol,
                                protocols, args.no_nvls, healthy))
            extra.update(reference_ratios(world, ms, extra))
        except Exception as ex:  # extras never block the headline line
            extra["extras_error"] = repr(ex)[:300]

    line = {
        "metric": "gemm_allreduce_tflops", "value": round(value, 2), "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "ours",
        "config": config_dict(M, N, K, world),
        "clocks": clocks,
        "e2e": {"value": round(flops / (e2e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms, 5),
                "steps": e2e_steps, "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": 128 * N * 2,
                "note": "input copied from pinned host memory every step (double-buffered, overlapping "
                        "the previous step's kernel); the first 128 of the 8192 result rows (1.6 % of the result) "
                        "are read back every step"},
        "gpu_launches": args.steps * 1,
        "extra": extra,
    }
    if rank == 0:
        print(json.dumps(line), file=REAL_STDOUT, flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def extras(torch, dist, impl, rank, world, dev, A, B, C, algo, flush, peaks, steps_main, protocol="push",
           protocols=("push",), no_nvls=False, healthy=None):
    """Comparison arms on the same box: our GEMM then one NCCL call (non-overlap), cuBLAS + NCCL,
    the counter-gated NCCL mechanism, and the GEMM+ReduceScatter+RMSNorm config."""
    from flashoverlap_b200 import ops
    from flashoverlap_b200.parallel import bootstrap
    from flashoverlap_b200.utils import config, layout

    out = {}
    steps, warm = max(20, min(steps_main, 100)), 5
    M, N = A.shape[0], B.shape[0]
    Cn = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    ms, _, _ = time_steps(torch, dist, world, lambda: impl.gemm_allreduce(A, B, Cn, algo), steps, warm, flush)
    out["nonoverlap_ourgemm_nccl_ms"] = round(ms, 5)
    base = bootstrap.make_baseline_impl(rank, world)
    ms, _, _ = time_steps(torch, dist, world, lambda: base.gemm_allreduce(A, B, Cn), steps, warm, flush)
    out["cublas_nccl_ms"] = round(ms, 5)
    # The two bare GEMMs are timed with the clock sampler as well: under the power cap the SM clock
    # each kernel sustains is what separates them.
    def brief(c):
        return None if not c else {"sm_mhz": c.get("sm_mhz"), "power_w_max": c.get("power_w_max"), "reasons": c.get("reasons")}

    smp = ClockSampler(dev.index) if rank == 0 else None
    ms, clk, _ = time_steps(torch, dist, world, lambda: base.cublas_gemm(A, B, Cn), steps, warm, flush, smp)
    out["cublas_gemm_only_ms"] = round(ms, 5)
    out["cublas_gemm_only_clocks"] = brief(clk)
    smp = ClockSampler(dev.index) if rank == 0 else None
    ms, clk, _ = time_steps(torch, dist, world, lambda: impl.cutlass_gemm(A, B, Cn, algo), steps, warm, flush, smp)
    out["our_gemm_only_ms"] = round(ms, 5)
    out["our_gemm_only_clocks"] = brief(clk)
    if world > 1:
        Dn = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)
        ms, _, _ = time_steps(torch, dist, world, lambda: impl.gemm_reducescatter_fused(A, B, Dn, algo), steps, warm, flush)
        out["fused_rs_same_shape_ms"] = round(ms, 5)
        ms, _, _ = time_steps(torch, dist, world, lambda: impl.gemm_allreduce_fused(A, B, C, algo), steps, warm, flush)
        out["fused_ar_natural_ms"] = round(ms, 5)
    if world > 1:
        cfg = config.default_solution(M, N, algo, wave_size=148 - 16)
        tiles = (M // cfg["BM"]) * (N // cfg["BN"])
        nw = layout.div_up(tiles, 148 - 16)
        groups = [nw // 4 + (1 if i < nw % 4 else 0) for i in range(4)] if nw >= 4 else [1] * nw
        cseg = layout.cseg_from_wave_groups(tiles, 148 - 16, groups)
        RA = layout.reorder_indices(tiles, cfg["hint"], device=dev)
        mm = torch.zeros(1, max(N // cfg["BN"], len(cseg)), device=dev, dtype=torch.int32)
        cseg_cpu = torch.tensor(cseg, dtype=torch.int32)
        cseg_gpu = cseg_cpu.to(dev)
        impl.set_option("mode", 1)
        try:
            ms, _, _ = time_steps(torch, dist, world,
                                  lambda: impl.gemm_allreduce_overlap(A, B, Cn, mm, RA, 1, cseg_cpu, cseg_gpu, algo, False),
                                  steps, warm, flush)
            out["gated_nccl_ms"] = round(ms, 5)
        finally:
            impl.set_option("mode", 0)

    # GEMM + ReduceScatter + RMSNorm (sequence-parallel o_proj shape).  Candidates: the fused
    # reduce-scatter (push or pull protocol) into the tile-contiguous shard followed by the fused
    # un-reorder+RMSNorm kernel, and the fused reduce-scatter whose reducers normalise each row
    # panel themselves (RMSNorm tail, push protocol); the fastest in a short probe is timed.
    from flashoverlap_b200.parallel import symm
    M2, N2, K2 = M_RS, N_RS, K_RS_TOTAL // world
    A2 = (torch.randn(M2, K2, device=dev) * 0.02).to(torch.bfloat16)
    B2 = (torch.randn(N2, K2, device=dev) * 0.02).to(torch.bfloat16)
    w = (1 + 0.02 * torch.randn(N2, device=dev)).to(torch.bfloat16)
    D = torch.empty(M2 // world, N2, device=dev, dtype=torch.bfloat16)
    Y = torch.empty_like(D)
    empty, empty_gpu = torch.empty(0, dtype=torch.int32), torch.empty(0, dtype=torch.int32, device=dev)
    rs_protocols = ["push"]
    if world > 1 and "pull" in protocols:
        try:
            symm.alloc_stage(impl, M2, N2, torch.bfloat16, multicast=not no_nvls)
            rs_protocols.append("pull")
        except Exception:
            pass
    rs_state = {}

    def rs_step(cand):
        a, proto, how = cand
        if a not in rs_state:
            c2 = config.default_solution(M2, N2, a)
            t2 = (M2 // c2["BM"]) * (N2 // c2["BN"])
            rs_state[a] = (c2, layout.reorder_indices(t2, c2["hint"], device=dev),
                           torch.zeros(1, N2 // c2["BN"], device=dev, dtype=torch.int32))
        c2, RA2, mm2 = rs_state[a]
        if world > 1:
            impl.set_option("stage_local", 1 if proto == "pull" else 0)
        if how == "tail":
            impl.gemm_reducescatter_rmsnorm_fused(A2, B2, Y, w, 1e-5, a)
        else:
            impl.gemm_reducescatter_overlap(A2, B2, D, D, mm2, RA2, empty_gpu, 1, empty, empty_gpu, a, False)
            torch.ops.flashoverlap_op.reorder_rmsnorm_eps(D, Y, w, c2["BM"] // world, c2["BN"], 1, RA2, 1e-5)

    rs_cands = [(a, pr, "norm_kernel") for pr in rs_protocols for a in (0, 1, 3)]
    if world > 1:
        rs_cands += [(a, "push", "tail") for a in (0, 1)]
    rs_cand, rs_probe = pick_algo(torch, dist, world, rs_step, rs_cands, flush, settle_seconds=0.2, check=healthy)
    ms, _, _ = time_steps(torch, dist, world, lambda: rs_step(rs_cand), steps, warm, flush)
    if world > 1:
        impl.set_option("stage_local", 1 if protocol == "pull" else 0)
    S2 = M2 * N2 * 2
    t_gemm = 2.0 * M2 * N2 * K2 / (peaks["bf16_tflops"] * 1e12)
    t_link = (S2 * (world - 1) / world) / (NVLINK_GBS * 1e9) if world > 1 else 0.0
    t_norm = 2.0 * (S2 / world) / (peaks["hbm_gbs"] * 1e9)
    rs = {"ms": round(ms, 5), "roofline_ms": round((max(t_gemm, t_link) + t_norm) * 1e3, 4), "M": M2, "N": N2, "K_per_rank": K2,
          "algo": rs_cand[0], "protocol": rs_cand[1], "rmsnorm": rs_cand[2],
          "probe": {f"{a}/{pr}/{how}": t for (a, pr, how), t in zip(rs_cands, rs_probe)}}
    rs["roofline_frac"] = round(rs["roofline_ms"] / ms, 4)
    C2 = torch.empty(M2, N2, device=dev, dtype=torch.bfloat16)

    def rs_base():
        base.gemm_reducescatter(A2, B2, C2, D)
        torch.ops.flashoverlap_op.rmsnorm(D, Y, w, 1e-5)

    msb, _, _ = time_steps(torch, dist, world, rs_base, steps, warm, flush)
    rs["cublas_nccl_rmsnorm_ms"] = round(msb, 5)
    rs["speedup_vs_cublas_nccl"] = round(msb / ms, 4)
    out["rs_rmsnorm"] = rs

    # Where the fused step's time goes (several ranks only): the depth of the push pipeline, and
    # the step with parts of the collective switched off (results are wrong in those runs; they
    # come last and nothing reads C afterwards).
    if world > 1:
        study = {}
        try:
            cfg_a = config.default_solution(M, N, algo)
            RA_a = layout.reorder_indices((M // cfg_a["BM"]) * (N // cfg_a["BN"]), cfg_a["hint"], device=dev)
            mm_a = torch.zeros(1, max(N // cfg_a["BN"], 8), device=dev, dtype=torch.int32)
            fused = lambda: impl.gemm_allreduce_overlap(A, B, C, mm_a, RA_a, 1, empty, empty_gpu, algo, False)
            for lag in (1, 2, 4):
                impl.set_option("push_lag", lag)
                ms, _, _ = time_steps(torch, dist, world, fused, steps, warm, flush)
                study[f"push_lag_{lag}_ms"] = round(ms, 5)
            impl.set_option("push_lag", 0)
            for bits, name in ((1, "no_reduction_traffic"), (2, "no_push_stores"), (3, "neither")):
                impl.set_option("diag", bits)
                ms, _, _ = time_steps(torch, dist, world, fused, steps, warm, flush)
                study[f"{name}_ms"] = round(ms, 5)
        except Exception as ex:
            study["error"] = repr(ex)[:200]
        finally:
            impl.set_option("push_lag", 0)
            impl.set_option("diag", 0)
        out["fused_step_study"] = study
    impl.check_status()
    return out


def reference_ratios(world, ms, extra):
    """Ratios against the reference arm's last run at this world size, when that arm has run on
    this machine (it leaves its JSON line in the git-ignored baseline/_ref)."""
    try:
        from baseline import reference_run
        with open(reference_run.last_run_path(world)) as f:
            ref = json.load(f)
    except Exception:
        return {}
    rx = ref.get("extra", {})
    out = {"reference_ms_per_step": ref.get("ms_per_step"), "reference_path": rx.get("path")}
    if ref.get("ms_per_step"):
        out["speedup_vs_reference_overlap"] = round(ref["ms_per_step"] / ms, 4)
    if rx.get("baseline_impl_ms"):
        out["reference_baseline_impl_ms"] = rx["baseline_impl_ms"]
        out["speedup_vs_reference_baseline_impl"] = round(rx["baseline_impl_ms"] / ms, 4)
    rs = extra.get("rs_rmsnorm")
    if rs and rx.get("rs_rmsnorm_ms"):
        rs["reference_rs_rmsnorm_ms"] = rx["rs_rmsnorm_ms"]
        rs["speedup_vs_reference"] = round(rx["rs_rmsnorm_ms"] / rs["ms"], 4)
    if rs and rx.get("rs_baseline_impl_ms"):
        rs["reference_rs_baseline_impl_ms"] = rx["rs_baseline_impl_ms"]
        rs["speedup_vs_reference_baseline_impl"] = round(rx["rs_baseline_impl_ms"] / rs["ms"], 4)
    return out


def run_reference(args):
    from baseline import reference_arm
    reference_arm.main(args)


def _claim_stdout():
    """Only the JSON line may reach stdout: libraries (NCCL prints its version there) are sent
    to stderr by pointing fd 1 at fd 2; the returned file object writes to the real stdout."""
    sys.stdout.flush()
    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return real


def main():
    global REAL_STDOUT
    REAL_STDOUT = _claim_stdout()
    sys.modules.setdefault("bench", sys.modules[__name__])   # `import bench` elsewhere must see this module
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-extra", action="store_true", help="skip the comparison arms")
    ap.add_argument("--no-nvls", action="store_true", help="no NVSwitch multicast: peer stores / peer loads only")
    ap.add_argument("--protocol", choices=["auto", "push", "pull"], default="auto",
                    help="fused-collective protocol; auto = the faster of the two in a short probe")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
