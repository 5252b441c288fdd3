"""Multi-GPU tests: one process per GPU (NCCL), fused kernels over real NVLink peer memory.

Skipped when fewer than two GPUs are visible; the same kernels' cross-rank protocol is covered
on one GPU by the loopback tests in test_gpu_kernels.py.
"""
import os

import pytest
import torch
import torch.distributed as dist

from tests._mp import run_ranks

pytestmark = pytest.mark.gpu


def _world():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    return 8 if n >= 8 else (4 if n >= 4 else 2)


def _rand(shape, dev, seed, scale=0.5, dt=torch.bfloat16):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dt).to(dev)


def _setup(rank, world):
    from flashoverlap_b200.parallel import bootstrap
    impl = bootstrap.make_overlap_impl(rank, world)
    impl.set_option("timeout_ms", 5000)
    return impl


def _fused_worker(rank, world):
    from flashoverlap_b200 import ops
    from flashoverlap_b200.utils import config, layout
    dev = torch.device("cuda", rank)
    impl = _setup(rank, world)
    res = {}
    for (M, N, K, algo) in ((1024, 2048, 512, 0), (2048, 1024, 256, 6), (2048, 2048, 512, 1), (2048, 1024, 256, 3)):
        p = config.algo_params(algo)
        BM, BN = p["BM"], p["BN"]
        tiles = (M // BM) * (N // BN)
        A, B = _rand((M, K), dev, 10 + rank), _rand((N, K), dev, 20 + rank)
        ref = A.float() @ B.float().t()
        dist.all_reduce(ref)
        tol = 0.02 * ref.abs().max().item() + 1e-3
        hint = layout.analytic_hint(M, N, BM, BN, p["raster"], p["rows_per_unit"])
        RA = layout.reorder_indices(tiles, hint, device=dev).reshape(M // BM, N // BN)
        mm = torch.zeros(1, N // BN, device=dev, dtype=torch.int32)
        e, eg = torch.empty(0, dtype=torch.int32), torch.empty(0, dtype=torch.int32, device=dev)
        cseg = torch.tensor([tiles // 3, tiles - tiles // 3], dtype=torch.int32)
        # all-reduce, reordered layout, symmetric output, per-tile flags; repeated calls
        C = impl.symm_empty([M, N], "bfloat16")
        for _ in range(3):
            C.fill_(float("nan"))
            torch.cuda.synchronize(); dist.barrier()
            impl.gemm_allreduce_overlap(A, B, C, mm, RA, 1, e, eg, algo, False)
        got = ops.unreorder(C, M, N, BM, BN, RA)
        res[f"ar_reordered_{algo}"] = (got.float() - ref).abs().max().item() / tol
        # wave groups + ordinary (non symmetric) output tensor
        C2 = torch.full((M, N), float("nan"), device=dev, dtype=torch.bfloat16)
        impl.gemm_allreduce_overlap(A, B, C2, mm, RA, 1, cseg, cseg.to(dev), algo, False)
        res[f"ar_groups_{algo}"] = (ops.unreorder(C2, M, N, BM, BN, RA).float() - ref).abs().max().item() / tol
        # natural layout
        C.fill_(float("nan")); torch.cuda.synchronize(); dist.barrier()
        impl.gemm_allreduce_fused(A, B, C, algo)
        res[f"ar_natural_{algo}"] = (C.float() - ref).abs().max().item() / tol
        # output with an NVSwitch multicast mapping (multimem.st broadcast) when the box offers one
        from flashoverlap_b200.parallel import symm
        Cm, used_mc = symm.alloc_allreduce_output(impl, (M, N), torch.bfloat16)
        for _ in range(2):
            Cm.fill_(float("nan")); torch.cuda.synchronize(); dist.barrier()
            impl.gemm_allreduce_fused(A, B, Cm, algo)
        torch.cuda.synchronize(); dist.barrier()
        res[f"ar_multicast_{algo}"] = (Cm.float() - ref).abs().max().item() / tol
        res["info_multicast"] = 1.0 if used_mc else 0.0
        # reduce-scatter, both ownership rules, both layouts
        for strided in (1, 0):
            impl.set_option("strided_rows", strided)
            rows = layout.owned_rows(M, BM, world, rank, bool(strided)).to(dev)
            D = torch.full((M // world, N), float("nan"), device=dev, dtype=torch.bfloat16)
            impl.gemm_reducescatter_overlap(A, B, D, D, mm, RA, eg, 1, e, eg, algo, False)
            got = ops.unreorder(D, M // world, N, BM // world, BN, RA)
            res[f"rs_reordered_{algo}_{strided}"] = (got.float() - ref[rows]).abs().max().item() / tol
            D.fill_(float("nan"))
            impl.gemm_reducescatter_fused(A, B, D, algo)
            res[f"rs_natural_{algo}_{strided}"] = (D.float() - ref[rows]).abs().max().item() / tol
        impl.set_option("strided_rows", 1)
    torch.cuda.synchronize()
    res["status"] = impl.read_status()[0]
    return res


def test_fused_allreduce_reducescatter_multi_gpu(lib):
    world = _world()
    for r in run_ranks(_fused_worker, world, "nccl"):
        assert r.pop("status") == 0
        print("multicast output used:", bool(r.pop("info_multicast")))
        for k, v in r.items():
            assert v <= 1.0, (k, v)


def _pull_worker(rank, world):
    """Pull protocol: partials staged in the producing rank's memory, owners fetch them."""
    from flashoverlap_b200.parallel import symm
    from flashoverlap_b200.utils import config, layout
    dev = torch.device("cuda", rank)
    impl = _setup(rank, world)
    impl.set_option("stage_local", 1)
    switch_reduce = True
    res = {"info_switch_reduce": 0.0}
    for (M, N, K, algo) in ((1024, 2048, 512, 0), (2048, 2048, 512, 1), (2048, 1024, 256, 3)):
        BM = config.algo_params(algo)["BM"]
        A, B = _rand((M, K), dev, 30 + rank), _rand((N, K), dev, 40 + rank)
        ref = A.float() @ B.float().t()
        dist.all_reduce(ref)
        tol = 0.02 * ref.abs().max().item() + 1e-3
        stagings = ["peer_loads"] + (["switch"] if switch_reduce else [])
        for how in stagings:
            if how == "switch":
                _, used = symm.alloc_stage(impl, M, N, torch.bfloat16)   # multimem.ld_reduce when `used`
                res["info_switch_reduce"] = 1.0 if used else 0.0
            C, _ = symm.alloc_allreduce_output(impl, (M, N), torch.bfloat16)
            for _ in range(3):
                C.fill_(float("nan")); torch.cuda.synchronize(); dist.barrier()
                impl.gemm_allreduce_fused(A, B, C, algo)
            torch.cuda.synchronize(); dist.barrier()
            res[f"ar_{how}_{algo}"] = (C.float() - ref).abs().max().item() / tol
            for strided in (1, 0):
                impl.set_option("strided_rows", strided)
                rows = layout.owned_rows(M, BM, world, rank, bool(strided)).to(dev)
                D = torch.full((M // world, N), float("nan"), device=dev, dtype=torch.bfloat16)
                for _ in range(2):
                    impl.gemm_reducescatter_fused(A, B, D, algo)
                torch.cuda.synchronize(); dist.barrier()
                res[f"rs_{how}_{algo}_{strided}"] = (D.float() - ref[rows]).abs().max().item() / tol
            impl.set_option("strided_rows", 1)
    res["status"] = impl.read_status()[0]
    return res


def test_pull_protocol_multi_gpu(lib):
    """Pull protocol over real NVLink: first with peer loads, then with the staging in
    multicast-mapped memory, where the owners' reducers sum with multimem.ld_reduce."""
    world = _world()
    for r in run_ranks(_pull_worker, world, "nccl"):
        assert r.pop("status") == 0
        print("switch-side reduction used:", bool(r.pop("info_switch_reduce")))
        for k, v in r.items():
            assert v <= 1.0, (k, v)


def _all2all_worker(rank, world):
    from flashoverlap_b200.utils import layout
    dev = torch.device("cuda", rank)
    impl = _setup(rank, world)
    res = {}
    M, N, K = 2048, 1024, 256
    g = torch.Generator().manual_seed(99)                          # same matrix on every rank
    mlen = torch.randint(0, M // (world - 1) + 1, (world, world), generator=g, dtype=torch.int32)
    for algo in (0, 1, 3):
        A, B = _rand((M, K), dev, 50 + rank), _rand((N, K), dev, 60 + rank)
        C = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        recv = int(mlen[:, rank].sum() - mlen[rank, rank])
        Dref = torch.full((max(recv, 1), N), float("nan"), device=dev, dtype=torch.bfloat16)
        impl.gemm_all2all(A, B, C, Dref, algo, mlen)              # GEMM, then grouped NCCL send/recv
        for symmetric in (True, False):
            D = impl.symm_empty([max(recv, 1), N], "bfloat16") if symmetric else torch.empty_like(Dref)
            for _ in range(3):
                D.fill_(float("nan"))
                impl.gemm_all2all_fused(A, B, D, algo, mlen)
            torch.cuda.synchronize(); dist.barrier()
            tol = 0.02 * Dref[:recv].float().abs().max().item() + 1e-3 if recv else 1.0
            err = (D[:recv].float() - Dref[:recv].float()).abs().max().item() if recv else 0.0
            res[f"a2a_{algo}_{int(symmetric)}"] = err / tol
    res["status"] = impl.read_status()[0]
    return res


def test_gemm_all2all_fused_multi_gpu(lib):
    world = _world()
    for r in run_ranks(_all2all_worker, world, "nccl"):
        assert r.pop("status") == 0
        for k, v in r.items():
            assert v <= 1.0, (k, v)


def _norm_tail_worker(rank, world):
    from flashoverlap_b200 import ops
    dev = torch.device("cuda", rank)
    impl = _setup(rank, world)
    res = {}
    for (M, N, K, algo) in ((1024, 2048, 512, 0), (2048, 2048, 512, 1), (2048, 4096, 256, 23)):
        A, B = _rand((M, K), dev, 70 + rank), _rand((N, K), dev, 80 + rank)
        w = (1 + 0.1 * _rand((N,), dev, 5, scale=1.0).float()).to(torch.bfloat16)
        D = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)
        impl.gemm_reducescatter_fused(A, B, D, algo)
        expect = ops.rmsnorm(D, w, 1e-5).float()
        Y = torch.full_like(D, float("nan"))
        for _ in range(3):
            impl.gemm_reducescatter_rmsnorm_fused(A, B, Y, w, 1e-5, algo)
        torch.cuda.synchronize(); dist.barrier()
        res[f"rs_norm_{algo}"] = (Y.float() - expect).abs().max().item() / (0.02 * expect.abs().max().item())
        # with the residual of a pre-norm block in between, both protocols
        for pull in (0, 1):
            impl.set_option("stage_local", pull)
            R0 = _rand((M // world, N), dev, 90 + rank, scale=2.0)
            R = R0.clone()
            Y2 = torch.full_like(D, float("nan"))
            for _ in range(2):
                R.copy_(R0)
                impl.gemm_reducescatter_add_rmsnorm_fused(A, B, R, Y2, w, 1e-5, algo)
            torch.cuda.synchronize(); dist.barrier()
            h_ref = (R0.float() + D.float()).to(torch.bfloat16)
            y_ref = ops.rmsnorm(h_ref, w, 1e-5).float()
            res[f"rs_add_h_{algo}_{pull}"] = (R.float() - h_ref.float()).abs().max().item() / (0.02 * h_ref.float().abs().max().item())
            res[f"rs_add_norm_{algo}_{pull}"] = (Y2.float() - y_ref).abs().max().item() / (0.02 * y_ref.abs().max().item())
        impl.set_option("stage_local", 0)
    res["status"] = impl.read_status()[0]
    return res


def test_reducescatter_rmsnorm_tail_multi_gpu(lib):
    world = _world()
    for r in run_ranks(_norm_tail_worker, world, "nccl"):
        assert r.pop("status") == 0
        for k, v in r.items():
            assert v <= 1.0, (k, v)


def _api_worker(rank, world):
    from flashoverlap_b200 import ops
    from flashoverlap_b200.parallel import bootstrap
    from flashoverlap_b200.utils import config, layout
    dev = torch.device("cuda", rank)
    impl = _setup(rank, world)
    base = bootstrap.make_baseline_impl(rank, world)
    res = {}
    M, N, K, algo = 1024, 2048, 256, 0
    p = config.algo_params(algo)
    BM, BN = p["BM"], p["BN"]
    tiles = (M // BM) * (N // BN)
    A, B = _rand((M, K), dev, 30 + rank), _rand((N, K), dev, 40 + rank)
    ref = A.float() @ B.float().t()
    dist.all_reduce(ref)
    tol = 0.03 * ref.abs().max().item() + 1e-3
    C = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    D = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)
    # non-overlapped paths (natural layout, contiguous shards)
    impl.gemm_allreduce(A, B, C, algo)
    res["gemm_allreduce"] = (C.float() - ref).abs().max().item() / tol
    impl.gemm_reducescatter(A, B, C, D, algo)
    lo = rank * (M // world)
    res["gemm_reducescatter"] = (D.float() - ref[lo:lo + M // world]).abs().max().item() / tol
    base.gemm_allreduce(A, B, C)
    res["baseline_allreduce"] = (C.float() - ref).abs().max().item() / tol
    base.gemm_reducescatter(A, B, C, D)
    res["baseline_reducescatter"] = (D.float() - ref[lo:lo + M // world]).abs().max().item() / tol
    # bare collectives
    x = torch.full((64, 256), float(rank + 1), device=dev, dtype=torch.bfloat16)
    impl.nccl_allreduce(x)
    res["nccl_allreduce"] = abs(x[0, 0].item() - world * (world + 1) / 2)
    x.fill_(float(rank + 1))
    impl.seg_allreduce(x, torch.tensor([1, 3], dtype=torch.int32), 4)
    res["seg_allreduce"] = abs(x[-1, -1].item() - world * (world + 1) / 2)
    x.fill_(1.0)
    impl.nccl_reducescatter(x)
    n = x.numel() // world
    res["nccl_reducescatter"] = abs(x.view(-1)[rank * n].item() - world)
    # counter-gated NCCL mechanism (the reference's scheme) on both collectives
    impl.set_option("mode", 1)
    wave = impl.get_option("sm_count") - impl.get_option("sm_margin")
    hint = layout.analytic_hint(M, N, BM, BN, p["raster"], p["rows_per_unit"])
    cseg = layout.cseg_from_wave_groups(tiles, max(1, min(wave, tiles // 2)), [1] * layout.div_up(tiles, max(1, min(wave, tiles // 2))))
    RA = layout.reorder_indices(tiles, hint, device=dev).reshape(M // BM, N // BN)
    mm = torch.zeros(1, max(N // BN, len(cseg)), device=dev, dtype=torch.int32)
    cseg_cpu = torch.tensor(cseg, dtype=torch.int32)
    for _ in range(2):
        C.fill_(float("nan"))
        impl.gemm_allreduce_overlap(A, B, C, mm, RA, 1, cseg_cpu, cseg_cpu.to(dev), algo, False)
    res["gated_allreduce"] = (ops.unreorder(C, M, N, BM, BN, RA).float() - ref).abs().max().item() / tol
    RE = layout.generate_row_mapping(M, N, BM, BN, cseg, world, device=dev)
    D.fill_(float("nan"))
    impl.gemm_reducescatter_overlap(A, B, C, D, mm, RA, RE, 1, cseg_cpu, cseg_cpu.to(dev), algo, False)
    got = ops.unreorder(D, M // world, N, BM // world, BN, RA)
    res["gated_reducescatter"] = (got.float() - ref[rank::world]).abs().max().item() / tol
    impl.set_option("mode", 0)
    # variable-size all-to-all on packed rows vs torch
    ml = torch.tensor([[(3 * i + 5 * j) % 7 + 1 for j in range(world)] for i in range(world)], dtype=torch.int32)
    send_rows = int(sum(ml[rank, j] for j in range(world) if j != rank))
    recv_rows = int(sum(ml[j, rank] for j in range(world) if j != rank))
    src = _rand((send_rows, 128), dev, 50 + rank)
    dst = torch.zeros(recv_rows, 128, device=dev, dtype=torch.bfloat16)
    impl.nccl_all2all(src, dst, ml)
    ins = [int(ml[rank, j]) if j != rank else 0 for j in range(world)]
    outs = [int(ml[j, rank]) if j != rank else 0 for j in range(world)]
    exp = torch.zeros_like(dst)
    dist.all_to_all_single(exp, src, output_split_sizes=outs, input_split_sizes=ins)
    res["nccl_all2all"] = (dst.float() - exp.float()).abs().max().item()
    dst2 = torch.zeros_like(dst)
    base.nccl_all2all(src, dst2, ml)
    res["baseline_all2all"] = (dst2.float() - exp.float()).abs().max().item()
    torch.cuda.synchronize()
    res["status"] = impl.read_status()[0]
    return res


def test_reference_api_multi_gpu(lib):
    world = _world()
    for r in run_ranks(_api_worker, world, "nccl"):
        assert r.pop("status") == 0
        for k, v in r.items():
            assert v <= 1.0, (k, v)


def _layer_worker(rank, world):
    from flashoverlap_b200.models import DecoderConfig, TPDecoderLayer
    dev = torch.device("cuda", rank)
    impl = _setup(rank, world)
    cfg = DecoderConfig(hidden=1024, ffn=2048, n_heads=8, n_kv_heads=8 if world > 2 else 2, head_dim=128)
    batch, seq = 2, 256
    T = batch * seq
    x_full = _rand((T, cfg.hidden), dev, 7, scale=1.0)
    outs = {}
    for name, mode, tail in (("nccl", "nccl", False), ("fused", "fused", False), ("fused_tail", "fused", True)):
        layer = TPDecoderLayer(cfg, rank, world, batch, seq, impl=mode, overlap_impl=impl, seed=3, fuse_norm=tail)
        rows = layer.shard_rows().to(dev)
        y = layer(x_full[rows])
        full = torch.zeros(T, cfg.hidden, device=dev, dtype=torch.float32)
        full[rows] = y.float()
        dist.all_reduce(full)
        outs[name] = full
    torch.cuda.synchronize()
    err = max((outs["nccl"] - outs["fused"]).abs().max().item(), (outs["nccl"] - outs["fused_tail"]).abs().max().item())
    return {"err": err, "scale": outs["nccl"].abs().max().item(), "status": impl.read_status()[0]}


def test_decoder_layer_fused_matches_nccl(lib):
    world = _world()
    for r in run_ranks(_layer_worker, world, "nccl"):
        assert r["status"] == 0
        assert r["err"] <= 0.03 * r["scale"] + 1e-2, r


def _timeout_worker(rank, world):
    """Rank 1 never launches: rank 0's kernel must give up within its bound, report a status and
    leave the context usable.  The failure is made on the host (a launch that does not happen)."""
    import time
    dev = torch.device("cuda", rank)
    impl = _setup(rank, world)
    M, N, K = 256, 512, 128
    A, B = _rand((M, K), dev, 1), _rand((N, K), dev, 2)
    C = impl.symm_empty([M, N], "bfloat16")
    out = {"elapsed": 0.0, "status": [0] * 8}
    # one complete call first: the symmetric staging memory is allocated collectively
    impl.gemm_allreduce_fused(A, B, C, 0)
    torch.cuda.synchronize(); dist.barrier()
    impl.set_option("timeout_ms", 300)
    if rank == 0:
        t = time.time()
        impl.gemm_allreduce_fused(A, B, C, 0)
        torch.cuda.synchronize()
        out["elapsed"] = time.time() - t
        out["status"] = impl.read_status()
        try:
            impl.check_status()
            out["raised"] = False
        except RuntimeError:
            out["raised"] = True
        out["alive"] = float(torch.ones(8, device=dev).sum().item())
    dist.barrier()
    # The ranks now disagree on the call number (rank 0 made a call that rank 1 never saw): every
    # later fused call would time out.  resync() - collective - brings them back in step.
    impl.set_option("timeout_ms", 5000)
    impl.resync()
    ref = A.float() @ B.float().t()
    dist.all_reduce(ref)
    for _ in range(2):
        C.fill_(float("nan")); torch.cuda.synchronize(); dist.barrier()
        impl.gemm_allreduce_fused(A, B, C, 0)
    torch.cuda.synchronize(); dist.barrier()
    out["after_resync_status"] = impl.read_status()[0]
    out["after_resync_err"] = (C.float() - ref).abs().max().item() / (0.02 * ref.abs().max().item() + 1e-3)
    return out


def test_missing_peer_times_out_with_status(lib):
    if (torch.cuda.device_count() if torch.cuda.is_available() else 0) < 2:
        pytest.skip("needs at least 2 GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    res = run_ranks(_timeout_worker, 2, "nccl")
    r0 = res[0]
    assert r0["status"][0] in (5, 6, 7), r0          # a cross-GPU wait gave up
    assert r0["raised"] and r0["alive"] == 8.0
    assert r0["elapsed"] < 10.0
    for r in res:
        assert r["after_resync_status"] == 0 and r["after_resync_err"] <= 1.0, r


def _rejected_call_worker(rank, world):
    """A fused call that the host rejects after the collective set-up (a trace buffer too small
    for the shape) must not advance the call number: the next call succeeds on every rank."""
    dev = torch.device("cuda", rank)
    impl = _setup(rank, world)
    M, N, K = 512, 1024, 128
    A, B = _rand((M, K), dev, 3 + rank), _rand((N, K), dev, 5 + rank)
    ref = A.float() @ B.float().t()
    dist.all_reduce(ref)
    C = impl.symm_empty([M, N], "bfloat16")
    impl.gemm_allreduce_fused(A, B, C, 0)
    torch.cuda.synchronize(); dist.barrier()
    impl.set_trace(torch.zeros(8, device=dev, dtype=torch.int64))      # far too small
    raised = False
    try:
        impl.gemm_allreduce_fused(A, B, C, 0)
    except RuntimeError as ex:
        raised = "trace buffer" in str(ex)
    impl.set_trace(torch.zeros(0, dtype=torch.int64))
    for _ in range(2):
        C.fill_(float("nan")); torch.cuda.synchronize(); dist.barrier()
        impl.gemm_allreduce_fused(A, B, C, 0)
    torch.cuda.synchronize(); dist.barrier()
    return {"raised": raised, "status": impl.read_status()[0],
            "err": (C.float() - ref).abs().max().item() / (0.02 * ref.abs().max().item() + 1e-3)}


def test_rejected_call_keeps_ranks_in_step(lib):
    world = _world()
    for r in run_ranks(_rejected_call_worker, world, "nccl"):
        assert r["raised"] and r["status"] == 0 and r["err"] <= 1.0, r


def _launch_skew_worker(rank, world):
    """Back-to-back fused calls with no barrier between them while, at every call, another rank
    reaches its launch tens of milliseconds late: the call-number handshake in the kernels must
    keep a fast rank's next call from overwriting staging or results a slow rank still needs.
    Operands change from call to call (exact power-of-two scales), so a stale slice would show."""
    import time
    from flashoverlap_b200.parallel import symm
    from flashoverlap_b200.utils import config, layout
    dev = torch.device("cuda", rank)
    impl = _setup(rank, world)
    M, N, K, algo = 2048, 2048, 512, 1
    BM = config.algo_params(algo)["BM"]
    A, B = _rand((M, K), dev, 50 + rank), _rand((N, K), dev, 60 + rank)
    ref = A.float() @ B.float().t()
    dist.all_reduce(ref)
    tol = 0.02 * ref.abs().max().item() + 1e-3
    rows = layout.owned_rows(M, BM, world, rank, True).to(dev)
    scales = (1.0, 4.0, 0.5, 2.0, 0.25, 8.0, 1.0, 2.0)
    res = {}
    for protocol in ("push", "pull"):
        impl.set_option("stage_local", 1 if protocol == "pull" else 0)
        C, _ = symm.alloc_allreduce_output(impl, (M, N), torch.bfloat16)
        D = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)
        torch.cuda.synchronize(); dist.barrier()
        snaps = []
        for i, s in enumerate(scales):
            if i % world == rank:
                time.sleep(0.03)                      # this rank launches late
            elif (i + 1) % world == rank:
                torch.cuda._sleep(20_000_000)         # this one is late on the device (~10 ms)
            As = A * s
            if i % 2 == 0:
                impl.gemm_allreduce_fused(As, B, C, algo)
                snaps.append((s, None, C.clone()))    # stream-ordered before this rank's next call
            else:
                D.fill_(float("nan"))
                impl.gemm_reducescatter_fused(As, B, D, algo)
                snaps.append((s, rows, D.clone()))
        torch.cuda.synchronize(); dist.barrier()
        worst = 0.0
        for s, r, got in snaps:
            want = ref * s if r is None else ref[r] * s
            worst = max(worst, (got.float() - want).abs().max().item() / (tol * s))
        res[f"skew_{protocol}"] = worst
    res["status"] = impl.read_status()[0]
    return res


def test_launch_skew_between_ranks(lib):
    world = _world()
    for r in run_ranks(_launch_skew_worker, world, "nccl"):
        assert r.pop("status") == 0
        for k, v in r.items():
            assert v <= 1.0, (k, v)
