"""Single-GPU numerics of every sm_100a kernel against plain PyTorch fp32 references."""
import time

import pytest
import torch

from flashoverlap_b200 import ops
from flashoverlap_b200.utils import config, layout


pytestmark = pytest.mark.gpu


def _rand(shape, dt, dev, scale=0.5):
    return (torch.randn(*shape, device=dev) * scale).to(dt)


def _tol(ref):
    return 0.02 * ref.abs().max().item() + 1e-3


@pytest.fixture(scope="module")
def impl(cuda):
    i = ops.OverlapImpl()
    i.nccl_init(0, 1, [0] * 16)
    i.cutlass_init()
    i.overlap_init()
    return i


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,dim", [(256, 1024), (384, 8192), (128, 16384), (130, 2048)])
def test_rmsnorm(cuda, dt, rows, dim):
    x = _rand((rows, dim), dt, cuda, 1.0)
    w = (1 + 0.02 * torch.randn(dim, device=cuda)).to(dt)
    y = ops.rmsnorm(x, w, 1e-6)
    ref = layout.rmsnorm_ref(x, w, 1e-6)
    assert (y.float() - ref.float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,dim,BM,BN,rldn", [(512, 2048, 128, 256, 1), (256, 1024, 64, 128, 1),
                                                 (512, 1024, 128, 128, 2), (128, 8192, 16, 256, 1)])
def test_reorder_roundtrip_and_reorder_rmsnorm(cuda, dt, rows, dim, BM, BN, rldn):
    tiles = (rows // BM) * (dim // BN)
    RA = torch.randperm(tiles, device=cuda, dtype=torch.int32)
    x = _rand((rows, dim), dt, cuda, 1.0)
    xr = ops.reorder(x, BM, BN, RA, rldn)
    assert torch.equal(xr.view(-1), layout.to_reordered(x, BM, BN, RA.cpu(), rldn).view(-1))
    assert torch.equal(ops.unreorder(xr, rows, dim, BM, BN, RA, rldn), x)
    w = (1 + 0.02 * torch.randn(dim, device=cuda)).to(dt)
    y = ops.reorder_rmsnorm(xr, rows, dim, w, BM, BN, RA, eps=1e-5, rldn=rldn)
    ref = layout.rmsnorm_ref(x, w, 1e-5)
    assert (y.float() - ref.float()).abs().max().item() <= 2e-2
    assert torch.equal(y, ops.rmsnorm(x, w, 1e-5))


def test_reference_signature_reorder_rmsnorm(cuda):
    """The 7-argument op of the reference (eps fixed at 1e-5)."""
    rows, dim, BM, BN = 256, 1024, 128, 256
    RA = torch.randperm(8, device=cuda, dtype=torch.int32).reshape(2, 4)
    x = _rand((rows, dim), torch.float16, cuda, 1.0)
    w = torch.ones(dim, device=cuda, dtype=torch.float16)
    xr = ops.reorder(x, BM, BN, RA)
    out = torch.empty_like(x)
    torch.ops.flashoverlap_op.reorder_rmsnorm(xr, out, w, BM, BN, 1, RA)
    assert (out.float() - layout.rmsnorm_ref(x, w, 1e-5).float()).abs().max().item() <= 2e-3


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K,algo", [(128, 256, 64, 0), (256, 512, 320, 1), (384, 384, 192, 2), (512, 256, 1024, 3),
                                        (1024, 2048, 512, 4), (2048, 1024, 1000, 8), (1280, 2304, 256, 12),
                                        (1024, 1024, 768, 16), (512, 4096, 128, 20), (2048, 2048, 2048, 6),
                                        (256, 256, 64, 1), (2048, 4096, 1024, 5), (4096, 2048, 512, 9),
                                        (8192, 8192, 256, 17), (1536, 1280, 384, 21),
                                        (512, 512, 64, 3), (2048, 2048, 1024, 7), (4096, 8192, 512, 19),
                                        (1024, 768, 320, 23), (512, 256, 192, 24), (2048, 4096, 512, 26),
                                        (4096, 2048, 1024, 29)])
def test_gemm_natural(cuda, impl, dt, M, N, K, algo):
    a, b = _rand((M, K), dt, cuda), _rand((N, K), dt, cuda)
    c = torch.full((M, N), float("nan"), device=cuda, dtype=dt)
    impl.cutlass_gemm(a, b, c, algo)
    ref = a.float() @ b.float().t()
    impl.check_status()
    assert (c.float() - ref).abs().max().item() <= _tol(ref)


def test_plain_gemm_and_row_kernels_replay_in_a_cuda_graph(cuda, impl):
    """The plain GEMM and the row kernels keep no per-call state on the host (tensor maps and
    parameters travel by value with the launch): captured once into a CUDA graph, they give the
    right result for operand values written after the capture."""
    M, N, K, algo = 512, 1024, 256, 1
    dt = torch.bfloat16
    a, b = _rand((M, K), dt, cuda), _rand((N, K), dt, cuda)
    w = (1 + 0.02 * torch.randn(N, device=cuda)).to(dt)
    c = torch.empty(M, N, device=cuda, dtype=dt)
    y = torch.empty_like(c)
    impl.cutlass_gemm(a, b, c, algo)                       # one-time set-up happens outside the capture
    ops.rmsnorm(c, w, 1e-5, out=y)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        impl.cutlass_gemm(a, b, c, algo)
        ops.rmsnorm(c, w, 1e-5, out=y)
    for _ in range(2):
        a.copy_(_rand((M, K), dt, cuda))
        b.copy_(_rand((N, K), dt, cuda))
        c.fill_(float("nan"))
        y.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        ref = a.float() @ b.float().t()
        assert (c.float() - ref).abs().max().item() <= _tol(ref)
        assert torch.equal(y, ops.rmsnorm(c, w, 1e-5))
    impl.check_status()


def test_gemm_rejects_bad_shapes(cuda, impl):
    a, b = _rand((100, 64), torch.bfloat16, cuda), _rand((256, 64), torch.bfloat16, cuda)
    with pytest.raises(RuntimeError):
        impl.cutlass_gemm(a, b, torch.empty(100, 256, device=cuda, dtype=torch.bfloat16), 0)
    a = _rand((128, 64), torch.bfloat16, cuda)
    with pytest.raises(RuntimeError):
        impl.cutlass_gemm(a, b.float(), torch.empty(128, 256, device=cuda, dtype=torch.bfloat16), 0)


@pytest.mark.parametrize("algo,rldn", [(0, 1), (6, 1), (0, 2), (1, 1), (5, 2), (3, 1), (7, 2)])
def test_gemm_reordered_signal_and_monitor(cuda, impl, algo, rldn):
    """World of one: gemm_allreduce_overlap is the reordered GEMM; monitor mode records each
    tile's completion rank exactly once."""
    M, N, K = 1024, 2048, 256
    p = config.algo_params(algo)
    tm, tn = M // p["BM"], N // p["BN"]
    RA = torch.randperm(tm * tn, device=cuda, dtype=torch.int32).reshape(tm, tn)
    a, b = _rand((M, K), torch.bfloat16, cuda), _rand((N, K), torch.bfloat16, cuda)
    c = torch.zeros(M, N, device=cuda, dtype=torch.bfloat16)
    mm = torch.zeros(tm + 1, tn, device=cuda, dtype=torch.int32)
    cseg = torch.tensor([tm * tn // 2, tm * tn - tm * tn // 2], dtype=torch.int32)
    impl.gemm_allreduce_overlap(a, b, c, mm, RA, rldn, cseg, cseg.to(cuda), algo, True)
    impl.check_status()
    ref = a.float() @ b.float().t()
    got = ops.unreorder(c, M, N, p["BM"], p["BN"], RA, rldn)
    assert (got.float() - ref).abs().max().item() <= _tol(ref)
    order = mm[1:].flatten().sort().values
    assert torch.equal(order, torch.arange(tm * tn, device=cuda, dtype=torch.int32))
    assert mm[0, tn - 1].item() == tm * tn


def test_analytic_hint_matches_monitor(cuda, impl):
    """With a persistent grid the completion wave of every tile is known by construction:
    tile at launch position p completes in wave p // grid (checked against the monitor)."""
    _check_hint(cuda, impl, 4)
    _check_hint(cuda, impl, 5)
    _check_hint(cuda, impl, 7)


def _check_hint(cuda, impl, algo):
    M, N, K = 4096, 4096, 512
    p = config.algo_params(algo)
    tm, tn = M // p["BM"], N // p["BN"]
    hint = layout.analytic_hint(M, N, p["BM"], p["BN"], p["raster"], p["rows_per_unit"])
    RA = torch.arange(tm * tn, device=cuda, dtype=torch.int32).reshape(tm, tn)   # identity: MM rows = natural ids
    a, b = _rand((M, K), torch.bfloat16, cuda), _rand((N, K), torch.bfloat16, cuda)
    c = torch.empty(M, N, device=cuda, dtype=torch.bfloat16)
    mm = torch.zeros(tm + 1, tn, device=cuda, dtype=torch.int32)
    e = torch.empty(0, dtype=torch.int32)
    impl.gemm_allreduce_overlap(a, b, c, mm, RA, 1, e, e.to(cuda), algo, True)
    order = mm[1:].flatten().cpu()
    grid = min(impl.get_option("sm_count") * p["mt"], tm * tn)   # tiles finished per wave
    waves_measured = (order // grid)
    waves_analytic = torch.empty(tm * tn, dtype=torch.long)
    waves_analytic[torch.tensor(hint)] = torch.arange(tm * tn) // grid
    # Tiles of the same CTA finish in order, so a tile can only be observed one wave away from
    # its analytic wave: when a fast CTA retires its next tile before a slow CTA has retired its
    # current one, the two swap completion ranks across the wave edge.  Nothing may be further off.
    diff = (waves_measured - waves_analytic).abs()
    assert diff.max().item() <= 1, diff.max().item()
    agree = (diff == 0).float().mean().item()
    assert agree > 0.9, agree


def test_wait_flag_completes_and_times_out(cuda):
    mm = torch.zeros(8, device=cuda, dtype=torch.int32)
    status = torch.zeros(8, device=cuda, dtype=torch.int32)
    mm[2] = 5
    ops.wait_flag(5, mm, 2, 500, status)
    torch.cuda.synchronize()
    assert status[0].item() == 0 and mm[2].item() == 0         # consumed and re-armed
    t = time.time()
    ops.wait_flag(7, mm, 3, 200, status)                        # nobody signals: bounded wait gives up
    torch.cuda.synchronize()
    assert 0.15 < time.time() - t < 5.0
    assert status[:4].tolist() == [8, 3, 0, 7]
    # the context is still healthy
    assert torch.ones(4, device=cuda).sum().item() == 4


def _loopback_case(cuda, comm_op, ws, M, N, K, algo, strided, natural, repeat=1, groups=None, dt=torch.bfloat16,
                   stage_local=False, epi_bufs=2):
    p = config.algo_params(algo)
    BM, BN = p["BM"], p["BN"]
    tiles = (M // BM) * (N // BN)
    A = [_rand((M, K), dt, cuda) for _ in range(ws)]
    B = [_rand((N, K), dt, cuda) for _ in range(ws)]
    full = sum(a.float() @ b.float().t() for a, b in zip(A, B))
    RA = torch.randperm(tiles, device=cuda, dtype=torch.int32)
    cseg = torch.tensor(groups, dtype=torch.int32, device=cuda) if groups else None
    rows = M if comm_op == "all_reduce" else M // ws
    out = [torch.full((rows, N), float("nan"), device=cuda, dtype=dt) for _ in range(ws)]
    st = ops.fused_loopback(comm_op, A, B, out, RA=RA, cseg=cseg, algo=algo, strided_rows=strided,
                            natural_out=natural, repeat=repeat, timeout_ms=2000, stage_local=stage_local,
                            epi_bufs=epi_bufs)
    assert all(s[0] == 0 for s in st), st
    for r in range(ws):
        if comm_op == "all_reduce":
            expect = full
            got = out[r] if natural else ops.unreorder(out[r], M, N, BM, BN, RA)
        else:
            expect = full[layout.owned_rows(M, BM, ws, r, strided).to(cuda)]
            got = out[r] if natural else ops.unreorder(out[r], M // ws, N, BM // ws, BN, RA)
        assert (got.float() - expect).abs().max().item() <= _tol(expect), (comm_op, r)


@pytest.mark.parametrize("comm_op", ["all_reduce", "reduce_scatter"])
@pytest.mark.parametrize("ws,algo,strided,natural", [(2, 0, True, False), (2, 0, False, True), (4, 2, True, True),
                                                     (4, 2, False, False)])
def test_fused_loopback(cuda, comm_op, ws, algo, strided, natural):
    """All ranks of the fused GEMM+collective kernel in one cooperative launch on one GPU."""
    _loopback_case(cuda, comm_op, ws, 1024, 2048, 512, algo, strided, natural)


@pytest.mark.parametrize("comm_op", ["all_reduce", "reduce_scatter"])
def test_fused_loopback_pull_protocol(cuda, comm_op):
    """Partials staged in the producing rank's own buffer, owners fetch and sum them."""
    _loopback_case(cuda, comm_op, 2, 1024, 2048, 512, 0, True, True, stage_local=True)
    _loopback_case(cuda, comm_op, 4, 1024, 2048, 256, 2, False, False, repeat=2, stage_local=True)
    _loopback_case(cuda, comm_op, 8, 2048, 2048, 256, 0, True, False, repeat=2, stage_local=True)
    _loopback_case(cuda, comm_op, 8, 1024, 1024, 128, 2, False, True, stage_local=True)
    _loopback_case(cuda, comm_op, 2, 2048, 2048, 256, 0, True, False, repeat=3, groups=[40, 50, 38],
                   dt=torch.float16, stage_local=True)


@pytest.mark.parametrize("ws,algo,dt", [(2, 0, torch.bfloat16), (4, 2, torch.bfloat16), (8, 0, torch.float16)])
def test_gemm_all2all_loopback(cuda, ws, algo, dt):
    """GEMM whose epilogue stores each row into its destination rank's receive buffer."""
    M, N, K = 1024, 1024, 256
    g = torch.Generator().manual_seed(ws)
    mlen = torch.randint(0, M // (ws - 1) + 1, (ws, ws), generator=g, dtype=torch.int32)
    mlen[0, 1 % ws] = 0                                           # an empty run
    A = [_rand((M, K), dt, cuda) for _ in range(ws)]
    B = [_rand((N, K), dt, cuda) for _ in range(ws)]
    C = [(a.float() @ b.float().t()) for a, b in zip(A, B)]
    want = layout.all2all_reference(C, mlen.tolist())
    out = [torch.full((max(1, w.shape[0]), N), float("nan"), device=cuda, dtype=dt) for w in want]
    st = ops.fused_loopback("all_to_all", A, B, out, algo=algo, repeat=2, timeout_ms=2000, mlen=mlen)
    assert all(s[0] == 0 for s in st), st
    for r in range(ws):
        n = want[r].shape[0]
        if n:
            assert (out[r][:n].float() - want[r]).abs().max().item() <= _tol(want[r]), r


@pytest.mark.parametrize("ws,algo,strided,dt", [(2, 0, True, torch.bfloat16), (4, 2, False, torch.bfloat16),
                                               (8, 0, True, torch.float16)])
def test_reducescatter_rmsnorm_tail_loopback(cuda, ws, algo, strided, dt):
    """Reducers that also normalise: out = rmsnorm(reduce_scatter(A B^T)) * w, no norm kernel."""
    M, N, K = 1024, 2048, 256
    BM = config.algo_params(algo)["BM"]
    A = [_rand((M, K), dt, cuda) for _ in range(ws)]
    B = [_rand((N, K), dt, cuda) for _ in range(ws)]
    w = (1 + 0.1 * torch.randn(N, device=cuda)).to(dt)
    full = sum(a.float() @ b.float().t() for a, b in zip(A, B))
    out = [torch.full((M // ws, N), float("nan"), device=cuda, dtype=dt) for _ in range(ws)]
    st = ops.fused_loopback("reduce_scatter", A, B, out, algo=algo, strided_rows=strided, natural_out=True,
                            repeat=2, timeout_ms=2000, norm_w=w, norm_eps=1e-5)
    assert all(s[0] == 0 for s in st), st
    for r in range(ws):
        shard = full[layout.owned_rows(M, BM, ws, r, strided).to(cuda)].to(dt)     # what the reducers round to
        expect = layout.rmsnorm_ref(shard, w, 1e-5).float()
        assert (out[r].float() - expect).abs().max().item() <= 0.03 * expect.abs().max().item(), r


def test_fused_loopback_timeline(cuda):
    """The tracing build of the fused kernel stamps every tile in order of its life cycle."""
    from flashoverlap_b200.utils import trace
    ws, M, N, K, algo = 2, 1024, 2048, 512, 0
    p = config.algo_params(algo)
    tiles = (M // p["BM"]) * (N // p["BN"])
    A = [_rand((M, K), torch.bfloat16, cuda) for _ in range(ws)]
    B = [_rand((N, K), torch.bfloat16, cuda) for _ in range(ws)]
    out = [torch.empty(M, N, device=cuda, dtype=torch.bfloat16) for _ in range(ws)]
    buf = trace.new_buffer(tiles, ws, cuda)
    st = ops.fused_loopback("all_reduce", A, B, out, algo=algo, natural_out=True, trace=buf)
    assert all(s[0] == 0 for s in st), st
    full = sum(a.float() @ b.float().t() for a, b in zip(A, B))
    assert (out[0].float() - full).abs().max().item() <= _tol(full)
    t = buf.cpu().view(ws, tiles, trace.SLOTS)
    assert (t[:, :, :7] > 0).all()
    for a, b in ((0, 1), (1, 2), (2, 3), (4, 5), (5, 6), (3, 5)):     # signalled before the owner sees it
        assert (t[:, :, b] >= t[:, :, a]).all(), (a, b)
    s = trace.summarize(buf, tiles, rank=1)
    assert s["reduce"]["tiles"] == tiles and s["span"]["us"] > 0


@pytest.mark.parametrize("comm_op", ["all_reduce", "reduce_scatter"])
def test_fused_loopback_four_chunk_buffers(cuda, comm_op):
    """Build with four epilogue chunk buffers: the push warp keeps three chunks of stores in flight."""
    _loopback_case(cuda, comm_op, 2, 1024, 2048, 512, 0, True, True, epi_bufs=4)
    _loopback_case(cuda, comm_op, 4, 1024, 2048, 256, 2, False, False, repeat=3, epi_bufs=4)
    _loopback_case(cuda, comm_op, 8, 2048, 2048, 256, 0, True, False, repeat=2, epi_bufs=4)
    _loopback_case(cuda, comm_op, 2, 2048, 2048, 128, 2, True, True, repeat=2, stage_local=True, epi_bufs=4)


def test_fused_loopback_eight_ranks(cuda):
    """Eight ranks (16 owned rows per tile each), 18 CTAs per rank, on one GPU."""
    _loopback_case(cuda, "all_reduce", 8, 2048, 2048, 256, 0, True, False, repeat=2)
    _loopback_case(cuda, "reduce_scatter", 8, 2048, 2048, 256, 2, True, True)
    _loopback_case(cuda, "reduce_scatter", 8, 1024, 1024, 128, 0, False, False)


def test_fused_loopback_repeat_groups_fp16(cuda):
    _loopback_case(cuda, "all_reduce", 2, 2048, 2048, 256, 0, True, False, repeat=3, groups=[40, 50, 38])
    _loopback_case(cuda, "reduce_scatter", 4, 2048, 2048, 256, 4, True, False, repeat=3)
    _loopback_case(cuda, "all_reduce", 2, 512, 1024, 128, 8, True, True, repeat=2, dt=torch.float16)
    # agrees with the CPU model of the protocol (same staging layout and ownership rules)
    from flashoverlap_b200.parallel import cpu_model
    torch.manual_seed(5)
    A = [_rand((256, 128), torch.bfloat16, cuda) for _ in range(2)]
    B = [_rand((512, 128), torch.bfloat16, cuda) for _ in range(2)]
    out = [torch.empty(128, 512, device=cuda, dtype=torch.bfloat16) for _ in range(2)]
    ops.fused_loopback("reduce_scatter", A, B, out, algo=0, strided_rows=True, natural_out=True)
    model = cpu_model.fused_collective([a.cpu() for a in A], [b.cpu() for b in B], 128, 256, "reduce_scatter")
    for r in range(2):
        assert (out[r].cpu().float() - model[r].float()).abs().max().item() <= 0.1


def test_world1_reference_api(cuda, impl):
    """Every reference method is callable on a single rank (collectives are identities)."""
    M, N, K = 256, 512, 128
    a, b = _rand((M, K), torch.bfloat16, cuda), _rand((N, K), torch.bfloat16, cuda)
    ref = a.float() @ b.float().t()
    c = torch.empty(M, N, device=cuda, dtype=torch.bfloat16)
    d = torch.empty(M, N, device=cuda, dtype=torch.bfloat16)
    impl.gemm_allreduce(a, b, c, 0)
    assert (c.float() - ref).abs().max().item() <= _tol(ref)
    impl.gemm_reducescatter(a, b, c, d, 0)
    assert torch.equal(c, d)
    impl.nccl_allreduce(c); impl.nccl_reducescatter(c)
    impl.seg_allreduce(c, torch.tensor([1, 1], dtype=torch.int32), 2)
    base = ops.BaselineImpl()
    base.nccl_init(0, 1, [0] * 16); base.cublas_init()
    base.gemm_allreduce(a, b, d)
    assert (d.float() - ref).abs().max().item() <= _tol(ref)
    base.cublas_gemm(a, b, d); base.nccl_allreduce(d); base.nccl_reducescatter(d)
    assert impl.read_status()[0] == 0


def test_overlap_call_rejects_short_index_arrays(cuda, impl):
    """RA, MM, cSEG are used as address offsets by the kernel: arrays that are too short for the
    shape are refused on the host, before any launch."""
    M, N, K, algo = 512, 1024, 128, 0
    tm, tn = M // 128, N // 256
    tiles = tm * tn
    a, b = _rand((M, K), torch.bfloat16, cuda), _rand((N, K), torch.bfloat16, cuda)
    c = torch.zeros(M, N, device=cuda, dtype=torch.bfloat16)
    RA = torch.arange(tiles, device=cuda, dtype=torch.int32)
    mm = torch.zeros(tm + 1, tn, device=cuda, dtype=torch.int32)
    e = torch.empty(0, dtype=torch.int32)
    eg = e.to(cuda)
    with pytest.raises(RuntimeError, match="RA has"):
        impl.gemm_allreduce_overlap(a, b, c, mm, RA[: tiles - 1], 1, e, eg, algo, False)
    with pytest.raises(RuntimeError, match="monitor mode MM needs"):
        impl.gemm_allreduce_overlap(a, b, c, mm[:1], RA, 1, e, eg, algo, True)
    bad = torch.tensor([tiles - 1, 2], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="cSEG_CPU sums to"):
        impl.gemm_allreduce_overlap(a, b, c, mm, RA, 1, bad, bad.to(cuda), algo, False)
    with pytest.raises(RuntimeError, match="differ in length"):
        impl.gemm_allreduce_overlap(a, b, c, mm, RA, 1, bad[:1], bad.to(cuda), algo, False)
    with pytest.raises(RuntimeError, match="out of range"):
        impl.gemm_allreduce_overlap(a, b, c, mm, RA, 1, e, eg, 999, False)
    with pytest.raises(RuntimeError, match="RA has"):
        impl.gemm_reducescatter_overlap(a, b, c, c, mm, RA[:2], eg, 1, e, eg, algo, False)
    impl.check_status()
    impl.gemm_allreduce_overlap(a, b, c, mm, RA, 1, e, eg, algo, False)      # the object is still usable
    ref = a.float() @ b.float().t()
    got = ops.unreorder(c, M, N, 128, 256, RA.reshape(tm, tn))
    assert (got.float() - ref).abs().max().item() <= _tol(ref)


def test_bad_ra_value_is_reported_not_followed(cuda):
    """A tile position outside [0, tiles) in RA: with option ``validate`` the host refuses the call;
    without it the kernel reports kStatusBadArgument, keeps every access inside the buffers (the
    tile is stored at its natural position instead) and the context stays usable."""
    i = ops.OverlapImpl()
    i.nccl_init(0, 1, [0] * 16)
    M, N, K, algo = 512, 1024, 128, 0
    tiles = (M // 128) * (N // 256)
    a, b = _rand((M, K), torch.bfloat16, cuda), _rand((N, K), torch.bfloat16, cuda)
    c = torch.zeros(M, N, device=cuda, dtype=torch.bfloat16)
    mm = torch.zeros(1, N // 256, device=cuda, dtype=torch.int32)
    e = torch.empty(0, dtype=torch.int32)
    RA = torch.arange(tiles, device=cuda, dtype=torch.int32)
    RA[3] = tiles + 7
    i.set_option("validate", 1)
    with pytest.raises(RuntimeError, match="not a tile position"):
        i.gemm_allreduce_overlap(a, b, c, mm, RA, 1, e, e.to(cuda), algo, False)
    dup = torch.arange(tiles, device=cuda, dtype=torch.int32)
    dup[5] = 4
    with pytest.raises(RuntimeError, match="not a permutation"):
        i.gemm_allreduce_overlap(a, b, c, mm, dup, 1, e, e.to(cuda), algo, False)
    i.set_option("validate", 0)
    i.gemm_allreduce_overlap(a, b, c, mm, RA, 1, e, e.to(cuda), algo, False)
    torch.cuda.synchronize()
    st = i.read_status()
    assert st[0] == 9 and st[1] == 1 and st[2] == 3 and st[3] == tiles + 7, st      # bad argument: RA[3]
    with pytest.raises(RuntimeError, match="bad argument"):
        i.check_status()
    i.reset_status()
    RA[3] = 3
    c.fill_(float("nan"))
    i.gemm_allreduce_overlap(a, b, c, mm, RA, 1, e, e.to(cuda), algo, False)
    i.check_status()
    ref = a.float() @ b.float().t()
    got = ops.unreorder(c, M, N, 128, 256, RA)
    assert (got.float() - ref).abs().max().item() <= _tol(ref)


def test_check_status_raises_with_decoded_message(cuda):
    """A device wait that runs out, written into an OverlapImpl's own status words: read_status
    returns the code and its arguments, check_status raises with the decoded text, reset_status
    clears it.  The failure is made on the host: a counter that nothing ever sets."""
    i = ops.OverlapImpl()
    i.nccl_init(0, 1, [0] * 16)
    i.set_option("timeout_ms", 50)
    mm = torch.zeros(4, device=cuda, dtype=torch.int32)
    mm[2] = 3
    i.wait_flag(3, mm, 2)                              # satisfied at once, counter reset by the wait
    torch.cuda.synchronize()
    i.check_status()
    assert mm[2].item() == 0
    t0 = time.time()
    i.wait_flag(3, mm, 1)                              # nothing sets counter 1: the wait gives up
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    st = i.read_status()
    assert st[0] == 8 and st[1] == 1, st               # kStatusTimeoutWaitKernel, counter index
    with pytest.raises(RuntimeError, match="counting wait kernel"):
        i.check_status()
    i.reset_status()
    i.check_status()
    with pytest.raises(RuntimeError, match="outside MM"):
        i.wait_flag(1, mm, 9)


@pytest.mark.parametrize("algo", [0, 1, 2, 3, 22, 25])
def test_plain_epilogues_agree(cuda, algo):
    """TMA tensor stores and per-thread stores must write the same bytes, in the row-major and the
    tile-contiguous layout (rLDN 1 and 2)."""
    i = ops.OverlapImpl()
    i.nccl_init(0, 1, [0] * 16)
    M, N, K = 1024, 2048, 192
    p = config.algo_params(algo)
    tm, tn = M // p["BM"], N // p["BN"]
    a, b = _rand((M, K), torch.bfloat16, cuda), _rand((N, K), torch.bfloat16, cuda)
    ref = a.float() @ b.float().t()
    e = torch.empty(0, dtype=torch.int32)
    outs = {}
    for tma in (1, 0):
        i.set_option("tma_out", tma)
        c = torch.full((M, N), float("nan"), device=cuda, dtype=torch.bfloat16)
        i.cutlass_gemm(a, b, c, algo)
        assert (c.float() - ref).abs().max().item() <= _tol(ref)
        outs[("nat", tma)] = c
        for rldn in (1, 2):
            RA = torch.randperm(tm * tn, device=cuda, dtype=torch.int32, generator=torch.Generator(device=cuda).manual_seed(rldn))
            mm = torch.zeros(tm + 1, tn, device=cuda, dtype=torch.int32)
            c2 = torch.full((M, N), float("nan"), device=cuda, dtype=torch.bfloat16)
            i.gemm_allreduce_overlap(a, b, c2, mm, RA.reshape(tm, tn), rldn, e, e.to(cuda), algo, True)
            got = ops.unreorder(c2, M, N, p["BM"], p["BN"], RA.reshape(tm, tn), rldn)
            assert (got.float() - ref).abs().max().item() <= _tol(ref)
            assert torch.equal(mm[1:].flatten().sort().values, torch.arange(tm * tn, device=cuda, dtype=torch.int32))
            outs[(rldn, tma)] = c2
    i.check_status()
    for key in ("nat", 1, 2):
        assert torch.equal(outs[(key, 1)], outs[(key, 0)]), key


@pytest.mark.parametrize("comm_op", ["all_reduce", "reduce_scatter"])
@pytest.mark.parametrize("ws,algo,strided", [(2, 0, True), (4, 2, False), (8, 0, True)])
def test_fused_loopback_pull_direct_stores(cuda, comm_op, ws, algo, strided):
    """Pull protocol whose epilogue threads store the partial tiles into the local staging
    themselves (the push warp only announces each tile); repeated calls reuse the staging."""
    M, N, K = 1024, 1024, 192
    A = [_rand((M, K), torch.bfloat16, cuda) for _ in range(ws)]
    B = [_rand((N, K), torch.bfloat16, cuda) for _ in range(ws)]
    full = sum(a.float() @ b.float().t() for a, b in zip(A, B))
    rows = M if comm_op == "all_reduce" else M // ws
    out = [torch.full((rows, N), float("nan"), device=cuda, dtype=torch.bfloat16) for _ in range(ws)]
    st = ops.fused_loopback(comm_op, A, B, out, algo=algo, strided_rows=strided, natural_out=True, repeat=3,
                            stage_local=True, pull_direct=True)
    assert all(s[0] == 0 for s in st), st
    for r in range(ws):
        if comm_op == "all_reduce":
            ref = full
        else:
            ref = full[layout.owned_rows(M, 128, ws, r, strided).to(cuda)]
        assert (out[r].float() - ref).abs().max().item() <= _tol(full), (comm_op, r)


@pytest.mark.parametrize("ws,algo,strided,pull,direct", [(2, 0, True, False, False), (4, 2, False, True, False),
                                                         (8, 0, True, True, True), (4, 0, True, False, False)])
def test_reducescatter_residual_rmsnorm_tail_loopback(cuda, ws, algo, strided, pull, direct):
    """R <- R + reduce_scatter(A B^T), Y <- rmsnorm(R) * w inside the fused kernel's reducers, with
    either protocol: compared with the unfused arithmetic on 16-bit tensors."""
    dt = torch.bfloat16
    M, N, K = 1024, 2048, 192
    A = [_rand((M, K), dt, cuda) for _ in range(ws)]
    B = [_rand((N, K), dt, cuda) for _ in range(ws)]
    w = (1 + 0.1 * torch.randn(N, device=cuda)).to(dt)
    full = sum(a.float() @ b.float().t() for a, b in zip(A, B))
    res0 = [_rand((M // ws, N), dt, cuda, 2.0) for _ in range(ws)]
    R = [r.clone() for r in res0]
    Y = [torch.full((M // ws, N), float("nan"), device=cuda, dtype=dt) for _ in range(ws)]
    st = ops.fused_loopback("reduce_scatter", A, B, R, algo=algo, strided_rows=strided, natural_out=True,
                            stage_local=pull, pull_direct=direct, norm_w=w, norm_eps=1e-5, norm_res=R, norm_out=Y)
    assert all(s[0] == 0 for s in st), st
    for r in range(ws):
        rows = layout.owned_rows(M, 128, ws, r, strided).to(cuda)
        h_ref = (res0[r].float() + full[rows].to(dt).float()).to(dt)
        assert (R[r].float() - h_ref.float()).abs().max().item() <= _tol(full), r
        y_ref = layout.rmsnorm_ref(R[r], w, 1e-5).float()
        assert (Y[r].float() - y_ref).abs().max().item() <= 0.02 * y_ref.abs().max().item() + 1e-3, r


@pytest.mark.parametrize("ws,algo", [(2, 0), (8, 2)])
def test_reducescatter_rmsnorm_tail_pull_loopback(cuda, ws, algo):
    """The RMSNorm tail with the pull protocol (partials staged locally, owners fetch them)."""
    dt = torch.bfloat16
    M, N, K = 1024, 1024, 192
    A = [_rand((M, K), dt, cuda) for _ in range(ws)]
    B = [_rand((N, K), dt, cuda) for _ in range(ws)]
    w = (1 + 0.1 * torch.randn(N, device=cuda)).to(dt)
    plain = [torch.empty(M // ws, N, device=cuda, dtype=dt) for _ in range(ws)]
    st = ops.fused_loopback("reduce_scatter", A, B, plain, algo=algo, natural_out=True)
    assert all(s[0] == 0 for s in st), st
    Y = [torch.full((M // ws, N), float("nan"), device=cuda, dtype=dt) for _ in range(ws)]
    st = ops.fused_loopback("reduce_scatter", A, B, Y, algo=algo, natural_out=True, stage_local=True, repeat=2,
                            norm_w=w, norm_eps=1e-5)
    assert all(s[0] == 0 for s in st), st
    for r in range(ws):
        y_ref = ops.rmsnorm(plain[r], w, 1e-5).float()
        assert (Y[r].float() - y_ref).abs().max().item() <= 0.02 * y_ref.abs().max().item() + 1e-3, r
