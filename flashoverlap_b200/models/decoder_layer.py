"""A Llama-style pre-norm decoder layer under tensor + sequence parallelism.

The reference ships no model beyond a row-parallel linear and an RMSNorm (example/*.py); this
layer is the end-to-end setting its two overlapped ops are meant for: the row-parallel
``o_proj`` and ``down_proj`` each end in a ReduceScatter along the token dimension followed by
an RMSNorm on the local tokens (Megatron sequence parallelism).  Everything that is not one of
those two ops uses stock PyTorch (cuBLAS matmul, SDPA, NCCL all-gather), as the reference has
nothing to offer there.

Two implementations of the same math:
  * ``impl="nccl"``:  ``matmul`` then ``dist.reduce_scatter_tensor`` - contiguous token shards;
  * ``impl="fused"``: one sm_100a kernel per projection that computes the tiles and
    reduce-scatters them over NVLink as they retire.  With the fused kernel every 128-token tile
    is split across the ranks (rank r owns tokens ``r*128/tp .. (r+1)*128/tp - 1`` of each
    tile), so an all-gather delivers the tokens tile-interleaved.  The gathered activations are
    NOT re-ordered: the column-parallel GEMMs do not care about row order, the (much narrower)
    QKV result is put into token order by the copy that splits it into heads, and SwiGLU writes
    its product straight into token order (``layout.tokens_as_gathered`` as the ``out=`` view).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..utils import layout

TILE_M = 128


@dataclass
class DecoderConfig:
    hidden: int = 8192
    ffn: int = 28672
    n_heads: int = 64
    n_kv_heads: int = 8
    head_dim: int = 128
    eps: float = 1e-5
    rope_theta: float = 500000.0

    @staticmethod
    def llama3_70b() -> "DecoderConfig":
        return DecoderConfig()

    @staticmethod
    def tiny() -> "DecoderConfig":
        return DecoderConfig(hidden=1024, ffn=2048, n_heads=8, n_kv_heads=2, head_dim=128)


def _rope(x: torch.Tensor, theta: float) -> torch.Tensor:
    # x: [B, H, S, D]
    B, H, S, D = x.shape
    pos = torch.arange(S, device=x.device, dtype=torch.float32)
    inv = theta ** (-torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D)
    ang = pos[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, None], ang.sin()[None, None]
    x1, x2 = x[..., 0::2].float(), x[..., 1::2].float()
    out = torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)
    return out.to(x.dtype)


class TPDecoderLayer(nn.Module):
    """Forward takes and returns the rank's token shard ``[T/tp, hidden]``.

    ``tokens`` (= batch * seq) must be a multiple of 128; ``overlap_impl`` is an initialised
    ``OverlapImpl`` (required for ``impl="fused"``).
    """

    def __init__(self, cfg: DecoderConfig, rank: int, world: int, batch: int, seq: int, impl: str = "fused",
                 overlap_impl=None, tp_group=None, dtype=torch.bfloat16, device="cuda", algo: int = 0,
                 seed: int = 0, fuse_norm: bool = False):
        super().__init__()
        assert impl in ("fused", "nccl")
        assert cfg.n_heads % world == 0 and cfg.n_kv_heads % world == 0 and cfg.ffn % world == 0
        assert (batch * seq) % TILE_M == 0 and TILE_M % world == 0
        self.cfg, self.rank, self.world, self.batch, self.seq = cfg, rank, world, batch, seq
        self.impl, self.ov, self.group, self.algo = impl, overlap_impl, tp_group, algo
        # impl="fused" only: o_proj's residual add and the RMSNorm that follows it run inside the
        # reduce-scatter kernel's reducers (gemm_reducescatter_add_rmsnorm_fused)
        self.fuse_norm = bool(fuse_norm) and impl == "fused" and world > 1
        if impl == "fused" and world > 1 and torch.device(device).type == "cuda":
            assert overlap_impl is not None, "impl='fused' needs an OverlapImpl"
            overlap_impl.set_option("strided_rows", 0)  # contiguous blocks inside each tile
        h, hd = cfg.hidden, cfg.head_dim
        self.q_local = cfg.n_heads // world
        self.kv_local = cfg.n_kv_heads // world
        self.ffn_local = cfg.ffn // world
        g = torch.Generator(device="cpu").manual_seed(seed + 1000 * rank)

        def w(o, i):
            return nn.Parameter((torch.randn(o, i, generator=g) * 0.02).to(dtype).to(device))

        self.wqkv = w((self.q_local + 2 * self.kv_local) * hd, h)   # column-parallel
        self.wo = w(h, self.q_local * hd)                           # row-parallel
        self.wgu = w(2 * self.ffn_local, h)                         # column-parallel (gate | up)
        self.wd = w(h, self.ffn_local)                              # row-parallel
        gn = torch.Generator(device="cpu").manual_seed(seed)        # norm weights are replicated
        self.attn_norm = nn.Parameter((1 + 0.02 * torch.randn(h, generator=gn)).to(dtype).to(device))
        self.mlp_norm = nn.Parameter((1 + 0.02 * torch.randn(h, generator=gn)).to(dtype).to(device))

    # ---- token <-> shard helpers -------------------------------------------------------------
    def shard_rows(self) -> torch.Tensor:
        """Global token indices held by this rank, in shard order."""
        T = self.batch * self.seq
        if self.impl == "fused" and self.world > 1:
            return layout.owned_rows(T, TILE_M, self.world, self.rank, strided=False)
        n = T // self.world
        return torch.arange(self.rank * n, (self.rank + 1) * n)

    def _norm(self, x, weight):
        if x.is_cuda:
            from .._build import load
            load()
            out = torch.empty_like(x)
            torch.ops.flashoverlap_op.rmsnorm(x, out, weight, self.cfg.eps)
            return out
        return layout.rmsnorm_ref(x, weight, self.cfg.eps)

    def _all_gather_tokens(self, x_sp: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x_sp
        n, h = x_sp.shape
        buf = torch.empty((self.world * n, h), dtype=x_sp.dtype, device=x_sp.device)
        dist.all_gather_into_tensor(buf, x_sp.contiguous(), group=self.group)
        return buf           # impl="fused": rows in gather order (rank-major), see _gathered

    @property
    def _gathered(self) -> bool:
        """True when all-gathered activations are tile-interleaved (fused ownership)."""
        return self.impl == "fused" and self.world > 1

    def _row_parallel(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """[T, k_local] @ weight[h, k_local]^T, summed over ranks, scattered over tokens."""
        T = x.shape[0]
        if self.world == 1:
            return torch.matmul(x, weight.t())
        if not x.is_cuda:
            # CPU ranks (tests of the layer's data flow): the same sums and the same token
            # ownership as the kernels, by an all-reduce and a row selection
            full = torch.matmul(x, weight.t())
            dist.all_reduce(full, group=self.group)
            return full[self.shard_rows()]
        out = torch.empty((T // self.world, weight.shape[0]), dtype=x.dtype, device=x.device)
        if self.impl == "fused":
            self.ov.gemm_reducescatter_fused(x.contiguous(), weight, out, self.algo)
        else:
            full = torch.matmul(x, weight.t())
            dist.reduce_scatter_tensor(out, full, group=self.group)
        return out

    # ---- forward -----------------------------------------------------------------------------
    def forward(self, x_sp: torch.Tensor) -> torch.Tensor:
        cfg, B, S, hd = self.cfg, self.batch, self.seq, self.cfg.head_dim
        # attention block
        xn = self._all_gather_tokens(self._norm(x_sp, self.attn_norm))          # [T, h]
        qkv = torch.matmul(xn, self.wqkv.t())
        if self._gathered:
            # token order for attention; this matrix is (q_local + 2 kv_local) * hd wide, not h
            qkv = layout.gathered_as_tokens(qkv, self.world, TILE_M).reshape(B * S, -1)
        q, k, v = qkv.split([self.q_local * hd, self.kv_local * hd, self.kv_local * hd], dim=-1)
        q = q.view(B, S, self.q_local, hd).transpose(1, 2)
        k = k.view(B, S, self.kv_local, hd).transpose(1, 2)
        v = v.view(B, S, self.kv_local, hd).transpose(1, 2)
        q, k = _rope(q, cfg.rope_theta), _rope(k, cfg.rope_theta)
        attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        attn = attn.transpose(1, 2).reshape(B * S, self.q_local * hd)
        if self.fuse_norm:
            # h = x + reduce_scatter(attn @ wo^T) and rmsnorm(h) * w in the kernel that reduces
            h_sp = x_sp.clone()
            hn_sp = torch.empty_like(h_sp)
            self.ov.gemm_reducescatter_add_rmsnorm_fused(attn.contiguous(), self.wo, h_sp, hn_sp, self.mlp_norm,
                                                         cfg.eps, self.algo)
            hn = self._all_gather_tokens(hn_sp)
        else:
            h_sp = x_sp + self._row_parallel(attn, self.wo)                    # [T/tp, h]
            hn = self._all_gather_tokens(self._norm(h_sp, self.mlp_norm))
        # MLP block
        gu = torch.matmul(hn, self.wgu.t())
        gate, up = gu.split([self.ffn_local, self.ffn_local], dim=-1)
        if self._gathered and not (torch.is_grad_enabled() and gu.requires_grad):
            # gate and up are in gather order; the product lands in token order, where the
            # row-parallel projection (and its token ownership) needs it
            act = torch.empty((B * S, self.ffn_local), dtype=gu.dtype, device=gu.device)
            dst = layout.tokens_as_gathered(act, self.world, TILE_M)
            torch.mul(F.silu(gate).view(dst.shape), up.view(dst.shape), out=dst)
        elif self._gathered:
            # out= is closed to autograd: the same placement as a copy of its own
            act = layout.gathered_as_tokens(F.silu(gate) * up, self.world, TILE_M).reshape(B * S, self.ffn_local)
        else:
            act = F.silu(gate) * up
        return h_sp + self._row_parallel(act, self.wd)
