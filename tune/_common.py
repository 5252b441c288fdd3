"""Shared pieces of the tuning CLIs: repository path set-up and the workload builders."""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from flashoverlap_b200.utils import config, layout  # noqa: E402

WARM_UP = 10
REP = 100


def str2bool(v: str) -> bool:
    """argparse ``type=bool`` turns every non-empty string into True (the reference has this bug
    at tune/search.py:515); this parses the usual spellings."""
    if isinstance(v, bool):
        return v
    return str(v).strip().lower() in ("1", "true", "yes", "y", "on")


def dtype_of(name: str):
    return torch.bfloat16 if name in ("bf16", "bfloat16") else torch.float16


def make_operands(M, N, K, dt, dev, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    A = (torch.randn(M, K, device=dev, generator=g) * 0.02).to(dt)
    B = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(dt)
    return A, B


class OverlapWorkload:
    """Everything a timed overlap call needs for one (shape, Algo, hint, cSeg)."""

    def __init__(self, impl, rank, world, M, N, K, algo, comm_op, dt, mode="fused", cseg=None, hint=None):
        dev = torch.device("cuda", torch.cuda.current_device())
        p = config.algo_params(algo)
        self.impl, self.world, self.comm_op, self.algo, self.mode = impl, world, comm_op, algo, mode
        self.BM, self.BN = p["BM"], p["BN"]
        self.M, self.N, self.K = M, N, K
        self.tiles = (M // self.BM) * (N // self.BN)
        self.hint = hint or layout.analytic_hint(M, N, self.BM, self.BN, p["raster"], p["rows_per_unit"])
        self.A, self.B = make_operands(M, N, K, dt, dev, seed=rank)
        self.RA = layout.reorder_indices(self.tiles, self.hint, device=dev).reshape(M // self.BM, N // self.BN)
        self.dev, self.dt = dev, dt
        if comm_op == "all_reduce" and world > 1 and mode == "fused":
            from flashoverlap_b200.parallel import symm
            self.C, _ = symm.alloc_allreduce_output(impl, (M, N), dt)
        else:
            self.C = torch.empty(M, N, device=dev, dtype=dt)
        self.D = torch.empty(M // world, N, device=dev, dtype=dt) if comm_op == "reduce_scatter" else None
        self.MM = torch.zeros(M // self.BM + 1, max(N // self.BN, 64), device=dev, dtype=torch.int32)
        self.set_cseg(cseg if cseg is not None else [self.tiles])

    def set_cseg(self, cseg):
        self.cseg = list(cseg)
        assert sum(self.cseg) == self.tiles
        if self.MM.shape[1] < len(self.cseg):
            self.MM = torch.zeros(self.M // self.BM + 1, len(self.cseg), device=self.dev, dtype=torch.int32)
        self.cseg_cpu = torch.tensor(self.cseg, dtype=torch.int32)
        self.cseg_gpu = self.cseg_cpu.to(self.dev)
        self.RE = (layout.generate_row_mapping(self.M, self.N, self.BM, self.BN, self.cseg, self.world, device=self.dev)
                   if (self.comm_op == "reduce_scatter" and self.mode == "gated")
                   else torch.zeros(1, dtype=torch.int32, device=self.dev))

    def run(self, monitor=False):
        self.impl.set_option("mode", 1 if self.mode == "gated" else 0)
        if self.comm_op == "all_reduce":
            self.impl.gemm_allreduce_overlap(self.A, self.B, self.C, self.MM, self.RA, 1, self.cseg_cpu, self.cseg_gpu,
                                             self.algo, monitor)
        else:
            tmp = self.C if self.mode == "gated" else self.D
            self.impl.gemm_reducescatter_overlap(self.A, self.B, tmp, self.D, self.MM, self.RA, self.RE, 1,
                                                 self.cseg_cpu, self.cseg_gpu, self.algo, monitor)

    def run_nonoverlap(self):
        if self.comm_op == "all_reduce":
            self.impl.gemm_allreduce(self.A, self.B, self.C, self.algo)
        else:
            self.impl.gemm_reducescatter(self.A, self.B, self.C, self.D, self.algo)
