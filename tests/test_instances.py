"""The kernel-instance generator (tool/generate_instances.py): the tables it writes are the ones
the package and the native library use, adding a kernel or a raster appends Algo numbers without
renumbering, and configurations that cannot fit the SM are refused."""
import copy
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gen():
    spec = importlib.util.spec_from_file_location("generate_instances", os.path.join(ROOT, "tool", "generate_instances.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_generated_tables_match_the_spec():
    gi = _gen()
    spec = gi.load_spec()
    from flashoverlap_b200.utils import _instances, config
    assert _instances.KERNELS == [(k["bn"], k["stages"], k["cta2"], k["mt"], k["stages_epi4"]) for k in spec["kernels"]]
    assert _instances.RASTERS == spec["rasters"]
    assert _instances.ALGOS == [tuple(a) for a in spec["algos"]]
    assert config.NUM_ALGOS == len(spec["algos"]) and config.NUM_KERNELS == len(spec["kernels"])
    inc = open(os.path.join(ROOT, "csrc", "gemm", "fo_gemm_instances.inc")).read()
    assert inc.count("FO_GEMM_KERNEL(") == len(spec["kernels"]) + 1        # + the comment line
    assert inc.count("FO_GEMM_ALGO(") == len(spec["algos"]) + 1
    # the first 24 Algos keep the historical numbering raster * 4 + kernel
    for a in range(24):
        assert tuple(spec["algos"][a]) == (a & 3, a >> 2)
    # every kernel fits the 227 KB of shared memory in both builds
    for k in spec["kernels"]:
        assert gi.smem_bytes(k["bn"], k["stages"], k["cta2"], k["mt"]) <= gi.SMEM_LIMIT
        assert gi.smem_bytes(k["bn"], k["stages_epi4"], k["cta2"], k["mt"], 4) <= gi.SMEM_LIMIT


def test_adding_kernels_and_rasters_appends_without_renumbering():
    gi = _gen()
    spec = copy.deepcopy(gi.load_spec())
    before = [tuple(a) for a in spec["algos"]]
    nk, nr = len(spec["kernels"]), len(spec["rasters"])
    idx = gi.add_kernel(spec, 128, 4, 0, 1)
    assert idx == nk and [tuple(a) for a in spec["algos"]][: len(before)] == before
    assert [tuple(a) for a in spec["algos"]][len(before):] == [(nk, r) for r in range(nr)]
    assert gi.add_kernel(spec, 128, 4, 0, 1) == idx and len(spec["kernels"]) == nk + 1      # already present
    r = gi.add_raster(spec, 32)
    assert r == nr and [tuple(a) for a in spec["algos"]][-(nk + 1):] == [(k, nr) for k in range(nk + 1)]
    assert spec["kernels"][idx]["stages_epi4"] >= 2
    for bad in (dict(bn=256, stages=9, cta2=0, mt=1), dict(bn=256, stages=4, cta2=0, mt=2), dict(bn=192, stages=2, cta2=0, mt=1),
                dict(bn=256, stages=1, cta2=0, mt=1)):
        with pytest.raises(ValueError):
            gi.add_kernel(copy.deepcopy(spec), **bad)
