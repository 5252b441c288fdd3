#!/usr/bin/env python
"""Generates the kernel-instance tables of the tcgen05 GEMM family from ``tool/instances.json``.

    python tool/generate_instances.py                                  # regenerate from the spec
    python tool/generate_instances.py --add-kernel bn=128,stages=8,cta2=1,mt=1
    python tool/generate_instances.py --list

The reference enumerates CUTLASS tile / stage / swizzle combinations and emits ``.inc`` files of
explicit instantiations, dispatch tables and ``AlgoDict.pt`` (tool/generate_instances.py:5-101);
its ``gen_config`` appends an Algo when a profiler row names a combination that is not built yet
and asks for a recompile (tune/gen_config.py:46-67).  Same idea here for one hand-written kernel
template: a *kernel* is a (BN, pipeline stages, CTA-pair mode, 128-row halves per CTA) tuple
- each one is a set of template instantiations - and an *Algo* is a (kernel, raster strip) pair.
The spec keeps the Algo list explicit, so adding a kernel or a raster appends new Algo numbers
and never renumbers the existing ones (tuned configs on disk stay valid).

Outputs (both tracked; rebuild the library after regenerating):
  csrc/gemm/fo_gemm_instances.inc        X-macro lists FO_GEMM_KERNEL(...) and FO_GEMM_ALGO(...)
  flashoverlap_b200/utils/_instances.py  the same tables for the Python side
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SPEC = os.path.join(ROOT, "tool", "instances.json")
INC = os.path.join(ROOT, "csrc", "gemm", "fo_gemm_instances.inc")
PY = os.path.join(ROOT, "flashoverlap_b200", "utils", "_instances.py")

BM, BK = 128, 64
SMEM_LIMIT = 227 * 1024
TMEM_COLS = 512
SIG_RING = 8   # slots of the ring between the push warp and the signal warp (kSigRing)


def smem_bytes(bn: int, stages: int, cta2: int, mt: int, epi: int = 2) -> int:
    """Dynamic shared memory of one instantiation (mirrors GemmSmem in fo_gemm_sm100.cuh)."""
    a = mt * BM * BK * 2
    b = (bn // 2 if cta2 else bn) * BK * 2
    bars = (2 * stages + 4 + 2 * epi + 2 * SIG_RING) * 8
    return stages * (a + b) + epi * BM * 128 + bars + 128 + 1024


def check_kernel(k: dict) -> None:
    bn, st, c2, mt = k["bn"], k["stages"], k["cta2"], k["mt"]
    if bn not in (128, 256):
        raise ValueError(f"bn={bn}: the kernel template is written for tile widths of 128 and 256 columns")
    if mt not in (1, 2) or (mt == 2 and not (c2 and bn == 256)):
        raise ValueError("mt=2 (two 128-row halves per CTA) needs cta2=1 and bn=256")
    if c2 not in (0, 1):
        raise ValueError("cta2 must be 0 or 1")
    if (bn // (2 if c2 else 1)) % 16:
        raise ValueError("each CTA's share of the B tile must be a multiple of 16 rows")
    if 2 * bn > TMEM_COLS:
        raise ValueError("two accumulators of bn columns must fit the 512 TMEM columns")
    if st < 2:
        raise ValueError("at least two pipeline stages")
    if smem_bytes(bn, st, c2, mt) > SMEM_LIMIT:
        raise ValueError(f"{smem_bytes(bn, st, c2, mt)} B of shared memory exceed {SMEM_LIMIT}")
    st4 = k.get("stages_epi4", 0)
    if st4 and smem_bytes(bn, st4, c2, mt, 4) > SMEM_LIMIT:
        raise ValueError(f"stages_epi4={st4}: the four-chunk-buffer build exceeds {SMEM_LIMIT} B")


def default_epi4_stages(bn: int, stages: int, cta2: int, mt: int) -> int:
    st4 = stages - 1
    while st4 >= 2 and smem_bytes(bn, st4, cta2, mt, 4) > SMEM_LIMIT:
        st4 -= 1
    return max(st4, 2)


def load_spec() -> dict:
    with open(SPEC) as f:
        spec = json.load(f)
    for k in spec["kernels"]:
        check_kernel(k)
    nk, nr = len(spec["kernels"]), len(spec["rasters"])
    seen = set()
    for a in spec["algos"]:
        if not (0 <= a[0] < nk and 0 <= a[1] < nr) or tuple(a) in seen:
            raise ValueError(f"bad or duplicate Algo entry {a}")
        seen.add(tuple(a))
    return spec


def save_spec(spec: dict) -> None:
    with open(SPEC, "w") as f:
        json.dump(spec, f, indent=1)
        f.write("\n")


def add_kernel(spec: dict, bn: int, stages: int, cta2: int, mt: int, stages_epi4: int = 0) -> int:
    """Appends a kernel (unless an identical one exists) and one Algo per raster; returns its index."""
    for i, k in enumerate(spec["kernels"]):
        if (k["bn"], k["stages"], k["cta2"], k["mt"]) == (bn, stages, cta2, mt):
            return i
    k = {"bn": bn, "stages": stages, "cta2": cta2, "mt": mt,
         "stages_epi4": stages_epi4 or default_epi4_stages(bn, stages, cta2, mt)}
    check_kernel(k)
    spec["kernels"].append(k)
    idx = len(spec["kernels"]) - 1
    for r in range(len(spec["rasters"])):
        spec["algos"].append([idx, r])
    return idx


def add_raster(spec: dict, strip: int) -> int:
    """Appends a raster strip width (0 = whole row panels) and one Algo per kernel."""
    if strip in spec["rasters"]:
        return spec["rasters"].index(strip)
    spec["rasters"].append(strip)
    r = len(spec["rasters"]) - 1
    for k in range(len(spec["kernels"])):
        spec["algos"].append([k, r])
    return r


def emit(spec: dict) -> None:
    ks, rs, al = spec["kernels"], spec["rasters"], spec["algos"]
    lines = ["// Generated by tool/generate_instances.py from tool/instances.json - do not edit by hand.",
             "// FO_GEMM_KERNEL(index, BN, stages, CTA pair, 128-row halves per CTA, stages of the",
             "//                four-chunk-buffer build)",
             "// FO_GEMM_ALGO(Algo, kernel index, raster strip width in N tiles; 0 = whole row panels)",
             "#ifdef FO_GEMM_KERNEL"]
    for i, k in enumerate(ks):
        lines.append(f"FO_GEMM_KERNEL({i}, {k['bn']}, {k['stages']}, {'true' if k['cta2'] else 'false'}, {k['mt']}, "
                     f"{k['stages_epi4']})")
    lines += ["#endif", "#ifdef FO_GEMM_ALGO"]
    for a, (k, r) in enumerate(al):
        lines.append(f"FO_GEMM_ALGO({a}, {k}, {rs[r]})")
    lines += ["#endif", ""]
    with open(INC, "w") as f:
        f.write("\n".join(lines))
    with open(PY, "w") as f:
        f.write('"""Generated by tool/generate_instances.py from tool/instances.json - do not edit by hand."""\n')
        f.write("# (BN, stages, CTA pair, 128-row halves per CTA, stages of the four-chunk-buffer build)\n")
        f.write("KERNELS = [\n" + "".join(
            f"    ({k['bn']}, {k['stages']}, {k['cta2']}, {k['mt']}, {k['stages_epi4']}),\n" for k in ks) + "]\n")
        f.write(f"RASTERS = {rs!r}\n")
        f.write("# Algo number -> (kernel index, raster index)\n")
        f.write("ALGOS = [\n" + "".join(f"    ({k}, {r}),\n" for k, r in al) + "]\n")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--add-kernel", default=None, metavar="bn=..,stages=..,cta2=..,mt=..[,stages_epi4=..]")
    ap.add_argument("--add-raster", type=int, default=None, metavar="STRIP")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--out-root", default=None, help="write the generated files under this directory instead of the repository")
    args = ap.parse_args()
    if args.out_root:
        global INC, PY
        INC = os.path.join(args.out_root, "csrc", "gemm", "fo_gemm_instances.inc")
        PY = os.path.join(args.out_root, "flashoverlap_b200", "utils", "_instances.py")
        os.makedirs(os.path.dirname(INC), exist_ok=True)
        os.makedirs(os.path.dirname(PY), exist_ok=True)
    spec = load_spec()
    changed = False
    if args.add_kernel:
        kv = dict(item.split("=") for item in args.add_kernel.split(","))
        n = len(spec["kernels"])
        idx = add_kernel(spec, int(kv["bn"]), int(kv["stages"]), int(kv.get("cta2", 0)), int(kv.get("mt", 1)),
                         int(kv.get("stages_epi4", 0)))
        changed = len(spec["kernels"]) != n
        print(f"kernel index {idx}" + (" (added)" if changed else " (already present)"))
    if args.add_raster is not None:
        n = len(spec["rasters"])
        add_raster(spec, args.add_raster)
        changed = changed or len(spec["rasters"]) != n
    if changed:
        save_spec(spec)
    emit(spec)
    if args.list or changed:
        for a, (k, r) in enumerate(spec["algos"]):
            kk = spec["kernels"][k]
            print(f"Algo {a:3d}: BN {kk['bn']:3d}  stages {kk['stages']}  cta_group {1 + kk['cta2']}  "
                  f"rows/CTA {128 * kk['mt']}  raster {spec['rasters'][r]}  smem {smem_bytes(kk['bn'], kk['stages'], kk['cta2'], kk['mt'])} B")
    print(f"wrote {os.path.relpath(INC, ROOT)} and {os.path.relpath(PY, ROOT)}: {len(spec['kernels'])} kernels, "
          f"{len(spec['algos'])} Algos" + ("; rebuild the library" if changed else ""))


if __name__ == "__main__":
    sys.exit(main())
