"""The on-disk tuning state: ``configs/m{M}n{N}k{K}_{gpu}.json``, ``AlgoDict.pt`` and the
bandwidth curves - same names and keys as the reference so configs remain interchangeable
in shape (tune/profile_config.py:57-72, tune/search.py:20-51, tune/bandwidth.py:111,
tool/generate_instances.py:40-45).

Stage 1 (``gen_config`` / ``profile_config``) writes lists of the 10 fastest GEMM configs:
``{"BM": [...], "BN": [...], "dur": [...], "Algo": [...]}``.  ``search`` rewrites the file with
scalars plus ``hint`` (natural tile ids in completion order), ``cSeg`` (tiles per wave group)
and ``rLDN``.  Keys this library adds (``tp``, ``comm_op``, ``dtype``, ``mode``) are optional
and ignored by readers that do not know them.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import torch

# Kernels, raster strips and the Algo list come from the generated table (tool/generate_instances.py
# writes it together with csrc/gemm/fo_gemm_instances.inc; tests/test_config.py checks it against
# the native table whenever the library is loaded).
from ._instances import ALGOS as _ALGOS, KERNELS as _KERNELS_FULL, RASTERS as _RASTERS

_KERNELS = [k[:4] for k in _KERNELS_FULL]      # (BN, stages, CTA pair, row halves per CTA)
NUM_KERNELS = len(_KERNELS)
NUM_ALGOS = len(_ALGOS)
BM = 128
BK = 64


def algo_kernel(algo: int) -> int:
    """Index of the kernel (tile configuration) an Algo runs."""
    if not 0 <= algo < NUM_ALGOS:
        raise ValueError(f"Algo {algo} out of range [0, {NUM_ALGOS})")
    return _ALGOS[algo][0]


def algo_with_kernel(algo: int, kernel: int) -> int:
    """The Algo that runs ``kernel`` with the raster of ``algo``."""
    r = _ALGOS[algo][1]
    for a, (k, rr) in enumerate(_ALGOS):
        if k == kernel and rr == r:
            return a
    raise ValueError(f"no Algo for kernel {kernel} with raster {_RASTERS[r]}")


def algo_params(algo: int) -> Dict[str, int]:
    if not 0 <= algo < NUM_ALGOS:
        raise ValueError(f"Algo {algo} out of range [0, {NUM_ALGOS})")
    k, r = _ALGOS[algo]
    bn, stages, cta2, mt = _KERNELS[k]
    return {"BM": BM, "BN": bn, "BK": BK, "stages": stages, "raster": _RASTERS[r], "cta2": cta2, "mt": mt,
            "rows_per_unit": (2 if cta2 else 1) * mt, "kernel": k}


def algo_tuple(algo: int) -> Tuple[int, ...]:
    """12-tuple key of AlgoDict, the slot meaning adapted to a tcgen05 kernel:
    (BM, BN, BK, UMMA_M, UMMA_N, UMMA_K, cta_group, accumulator stages, epilogue chunk,
    pipeline stages, raster strip, split-K)."""
    p = algo_params(algo)
    return (p["BM"] * p["mt"], p["BN"], p["BK"], 128 * (1 + p["cta2"]), p["BN"], 16, 1 + p["cta2"], 3 - p["mt"], 64,
            p["stages"], p["raster"], 1)


def algo_dict() -> Dict[Tuple[int, ...], int]:
    return {algo_tuple(a): a for a in range(NUM_ALGOS)}


def default_config_dir() -> Path:
    return Path(os.environ.get("FLASHOVERLAP_CONFIG_DIR", Path(__file__).resolve().parents[2] / "configs"))


def save_algo_dict(path: Optional[os.PathLike] = None) -> Path:
    path = Path(path) if path else default_config_dir() / "AlgoDict.pt"
    path.parent.mkdir(parents=True, exist_ok=True)
    torch.save(algo_dict(), path)
    return path


def gpu_tag(name: Optional[str] = None) -> str:
    """"NVIDIA B200" -> "b200" (characters 7..10 of the device name, lower case)."""
    if name is None:
        name = torch.cuda.get_device_properties(0).name if torch.cuda.is_available() else "NVIDIA B200"
    return name[7:11].lower().strip() or "gpu"


def config_path(M: int, N: int, K: int, gpu: Optional[str] = None, directory: Optional[os.PathLike] = None) -> Path:
    d = Path(directory) if directory else default_config_dir()
    return d / f"m{M}n{N}k{K}_{gpu or gpu_tag()}.json"


def bandwidth_path(comm_op: str, world_size: int, directory: Optional[os.PathLike] = None) -> Path:
    d = Path(directory) if directory else default_config_dir()
    return d / f"bandwidth_{comm_op}_tp{world_size}.pt"


def load_config(path: os.PathLike) -> dict:
    with open(path) as f:
        return json.load(f)


def save_stage1(path: os.PathLike, BMs: Sequence[int], BNs: Sequence[int], durs: Sequence[float],
                algos: Sequence[int]) -> None:
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as f:
        json.dump({"BM": list(BMs), "BN": list(BNs), "dur": list(durs), "Algo": list(algos)}, f, indent=4)


def save_solution(path: os.PathLike, BM_: int, BN: int, dur: float, algo: int, hint: Sequence[int],
                  cseg: Sequence[int], rldn: int = 1, **extra) -> None:
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    data = {"BM": int(BM_), "BN": int(BN), "dur": float(dur), "Algo": int(algo),
            "hint": [int(h) for h in hint], "cSeg": [int(c) for c in cseg], "rLDN": int(rldn)}
    data.update(extra)
    with open(path, "w") as f:
        json.dump(data, f, indent=4)


def is_tuned(cfg: dict) -> bool:
    return "hint" in cfg and "cSeg" in cfg and not isinstance(cfg.get("Algo"), list)


def matches(cfg: dict, tp: Optional[int] = None, comm_op: Optional[str] = None, mode: Optional[str] = None) -> bool:
    """Whether a tuned config was searched for this use.  The file name carries only (M, N, K,
    gpu); ``search`` also records the world size, the collective and the overlap mechanism the
    grouping was tuned for.  A key the file does not carry (a config written by the reference's
    tools) matches anything; a key it carries must agree with the call."""
    for key, want in (("tp", tp), ("comm_op", comm_op), ("mode", mode)):
        if want is not None and key in cfg and cfg[key] != want:
            return False
    return True


def load_tuned(M: int, N: int, K: int, tp: Optional[int] = None, comm_op: Optional[str] = None,
               mode: Optional[str] = None, gpu: Optional[str] = None,
               directory: Optional[os.PathLike] = None, warn: bool = True) -> Optional[dict]:
    """The tuned config of a shape if there is one AND it was tuned for this world size,
    collective and mechanism; otherwise None (callers then fall back to ``default_solution``).
    A config tuned for the counter-gated all-reduce is never silently used for the fused
    reduce-scatter of the same shape."""
    path = config_path(M, N, K, gpu, directory)
    if not path.exists():
        return None
    cfg = load_config(path)
    if not is_tuned(cfg):
        return None
    if not matches(cfg, tp, comm_op, mode):
        if warn:
            import warnings
            have = {k: cfg.get(k) for k in ("tp", "comm_op", "mode") if k in cfg}
            warnings.warn(f"{path} was tuned for {have}, not for tp={tp} comm_op={comm_op} mode={mode}: ignored")
        return None
    return cfg


def default_solution(M: int, N: int, algo: int = 0, wave_size: int = 148, groups: Optional[List[int]] = None) -> dict:
    """A usable config without any tuning run: analytic hint and one wave per group."""
    from . import layout
    p = algo_params(algo)

    def fits(k):
        bn, _, cta2, mt = _KERNELS[k]
        return N % bn == 0 and M % ((2 if cta2 else 1) * mt * BM) == 0

    if not fits(p["kernel"]):
        # nearest kernel that divides the shape: CTA pairs, then one CTA per 128 x 256 tile, then BN = 128
        for k in (1, 0, 2):
            if fits(k):
                algo = algo_with_kernel(algo, k)
                p = algo_params(algo)
                break
    tiles = (M // p["BM"]) * (N // p["BN"])
    hint = layout.analytic_hint(M, N, p["BM"], p["BN"], p["raster"], p["rows_per_unit"])
    nw = layout.div_up(tiles, wave_size)
    cseg = layout.cseg_from_wave_groups(tiles, wave_size, groups or [1] * nw)
    return {"BM": p["BM"], "BN": p["BN"], "dur": 0.0, "Algo": algo, "hint": hint, "cSeg": cseg, "rLDN": 1}
