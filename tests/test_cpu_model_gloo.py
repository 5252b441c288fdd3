"""Semantic check of the overlap pipeline on CPU with 2 gloo ranks.

Per-rank A[256,512], B[512,1024] fp32 ~N(0, 1/512), seed = rank; C = A @ B, sum-all-reduced (and
separately reduce-scattered along M); RMSNorm over N=1024 with weight ~N(1, 0.02), eps 1e-6;
compared with the unfused matmul -> dist collective -> rms_norm at atol 1e-4.
"""
import torch
import torch.distributed as dist

from flashoverlap_b200.parallel import cpu_model
from flashoverlap_b200.utils import layout
from tests._mp import run_ranks

M, K, N, BM, BN, EPS = 256, 512, 1024, 128, 256, 1e-6


def _operands(rank):
    g = torch.Generator().manual_seed(rank)
    A = torch.randn(M, K, generator=g) * (1.0 / 512) ** 0.5
    Bt = torch.randn(K, N, generator=g) * (1.0 / 512) ** 0.5     # B[512,1024]
    gw = torch.Generator().manual_seed(1234)
    w = 1.0 + 0.02 * torch.randn(N, generator=gw)
    return A, Bt.t().contiguous(), w                               # weight layout [N, K]


def _worker(rank, world):
    A, B, w = _operands(rank)
    tm, tn = M // BM, N // BN
    hint = layout.raster_order(tm, tn, 2)
    cseg = [3, 5]
    RA = layout.reorder_indices(tm * tn, hint)
    # unfused reference
    C = A @ B.t()
    ar = C.clone()
    dist.all_reduce(ar)
    y_ar_ref = layout.rmsnorm_ref(ar, w, EPS)
    shard = torch.empty(M // world, N)
    dist.reduce_scatter_tensor(shard, layout.reorder_rows_by_world_size(C, world).contiguous())
    y_rs_ref = layout.rmsnorm_ref(shard, w, EPS)
    # overlap pipeline (counter-gated model): per-group collectives on the reordered buffer
    buf = cpu_model.gated_allreduce(A, B, BM, BN, hint, cseg)
    y_ar = layout.reorder_rmsnorm_ref(buf, M, N, BM, BN, RA, w, EPS)
    d = cpu_model.gated_reducescatter(A, B, BM, BN, hint, cseg)
    y_rs = layout.reorder_rmsnorm_ref(d, M // world, N, BM // world, BN, RA, w, EPS)
    return {"ar": (y_ar - y_ar_ref).abs().max().item(), "rs": (y_rs - y_rs_ref).abs().max().item(),
            "y_ar": y_ar, "C": C}


def test_gated_pipeline_matches_unfused_on_gloo():
    res = run_ranks(_worker, 2, "gloo")
    for r in res:
        assert r["ar"] < 1e-4, r["ar"]
        assert r["rs"] < 1e-4, r["rs"]
    assert torch.equal(res[0]["y_ar"], res[1]["y_ar"])


def test_fused_protocol_model_matches_sum():
    """Single-process model of the fused kernels' push/reduce protocol (all ownership modes)."""
    ops = [_operands(r) for r in range(2)]
    A, B = [o[0] for o in ops], [o[1] for o in ops]
    full = sum(a @ b.t() for a, b in zip(A, B))
    RA = torch.randperm((M // BM) * (N // BN), dtype=torch.int32)
    for strided in (True, False):
        outs = cpu_model.fused_collective(A, B, BM, BN, "all_reduce", strided=strided)
        assert all(torch.allclose(o, full, atol=1e-5) for o in outs)
        outs = cpu_model.fused_collective(A, B, BM, BN, "all_reduce", strided=strided, RA=RA, natural_out=False)
        assert torch.allclose(layout.from_reordered(outs[1], M, N, BM, BN, RA), full, atol=1e-5)
        outs = cpu_model.fused_collective(A, B, BM, BN, "reduce_scatter", strided=strided)
        for r, o in enumerate(outs):
            assert torch.allclose(o, full[layout.owned_rows(M, BM, 2, r, strided)], atol=1e-5)
        outs = cpu_model.fused_collective(A, B, BM, BN, "reduce_scatter", strided=strided, RA=RA, natural_out=False)
        for r, o in enumerate(outs):
            got = layout.from_reordered(o, M // 2, N, BM // 2, BN, RA)
            assert torch.allclose(got, full[layout.owned_rows(M, BM, 2, r, strided)], atol=1e-5)


def _decoder_layer_worker(rank, world):
    """The TP decoder layer's data flow on CPU ranks: the `fused` token ownership (every 128-token
    tile split across the ranks, activations gathered tile-interleaved and never re-ordered,
    SwiGLU written into token order through a strided view) against the `nccl` one (contiguous
    token shards).  Same weights, fp32."""
    from flashoverlap_b200.models import DecoderConfig, TPDecoderLayer
    cfg = DecoderConfig(hidden=256, ffn=512, n_heads=4, n_kv_heads=2, head_dim=32)
    batch, seq = 2, 128
    T = batch * seq
    g = torch.Generator().manual_seed(11)
    x_full = torch.randn(T, cfg.hidden, generator=g)
    outs = {}
    with torch.no_grad():
        for mode in ("nccl", "fused"):
            layer = TPDecoderLayer(cfg, rank, world, batch, seq, impl=mode, dtype=torch.float32, device="cpu", seed=3)
            rows = layer.shard_rows()
            full = torch.zeros(T, cfg.hidden)
            full[rows] = layer(x_full[rows])
            dist.all_reduce(full)
            outs[mode] = full
    return {"err": (outs["nccl"] - outs["fused"]).abs().max().item(), "scale": outs["nccl"].abs().max().item(),
            "interleaved": bool((rows[:64] != torch.arange(rank * (T // world), rank * (T // world) + 64)).any()) if rank else True}


def test_decoder_layer_fused_token_ownership_matches_contiguous_shards():
    for r in run_ranks(_decoder_layer_worker, 2, "gloo", timeout_s=120):
        assert r["interleaved"]
        assert r["err"] <= 1e-4 * max(1.0, r["scale"]), r
