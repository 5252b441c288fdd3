"""Config files and the Algo table (CPU)."""
import json

import torch

from flashoverlap_b200.utils import config


def test_algo_table_matches_native(lib):
    flat = list(torch.ops.flashoverlap_op.algo_table())
    assert len(flat) == 7 * config.NUM_ALGOS
    for a in range(config.NUM_ALGOS):
        p = config.algo_params(a)
        assert tuple(flat[7 * a:7 * a + 7]) == (p["BM"], p["BN"], p["BK"], p["stages"], p["raster"], p["cta2"], p["mt"])


def test_algo_dict_roundtrip(tmp_path):
    d = config.algo_dict()
    assert len(d) == config.NUM_ALGOS and all(len(k) == 12 for k in d)
    path = config.save_algo_dict(tmp_path / "AlgoDict.pt")
    assert torch.load(path, weights_only=False) == d


def test_config_names_and_stages(tmp_path):
    assert config.gpu_tag("NVIDIA B200") == "b200"
    assert config.gpu_tag("NVIDIA A800-SXM4-80GB") == "a800"
    p = config.config_path(4096, 8192, 8192, "b200", tmp_path)
    assert p.name == "m4096n8192k8192_b200.json"
    config.save_stage1(p, [128] * 10, [256] * 10, list(range(10)), list(range(10)))
    c = config.load_config(p)
    assert not config.is_tuned(c) and len(c["Algo"]) == 10
    config.save_solution(p, 128, 256, 0.5, 4, [1, 0], [1, 1], tp=2, comm_op="all_reduce")
    c = json.load(open(p))
    assert config.is_tuned(c) and c["rLDN"] == 1 and c["hint"] == [1, 0] and c["cSeg"] == [1, 1] and c["tp"] == 2
    assert config.bandwidth_path("all_reduce", 8, tmp_path).name == "bandwidth_all_reduce_tp8.pt"


def test_default_solution_is_consistent():
    c = config.default_solution(1024, 2048, algo=4)
    tiles = (1024 // c["BM"]) * (2048 // c["BN"])
    assert sorted(c["hint"]) == list(range(tiles)) and sum(c["cSeg"]) == tiles
    c = config.default_solution(1024, 2048 + 128, algo=0)      # N not a multiple of 256 -> BN 128
    assert c["BN"] == 128 and config.algo_kernel(c["Algo"]) == 2
    c = config.default_solution(768, 2048, algo=3)             # M not a multiple of 512 -> plain CTA pairs
    assert config.algo_kernel(c["Algo"]) == 1 and sorted(c["hint"]) == list(range((768 // 128) * (2048 // 256)))
    c = config.default_solution(1024, 2048, algo=7)            # two halves per CTA: units of 4 tile rows
    assert config.algo_kernel(c["Algo"]) == 3 and c["hint"][:4] == [0, 8, 16, 24]


def test_gen_config_csv_rows_map_back_to_algos(tmp_path, monkeypatch):
    """tune/gen_config.py: a CSV row that names a kernel of the table yields its Algo index."""
    import csv
    import importlib
    import os
    import sys

    tune_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tune")
    monkeypatch.syspath_prepend(tune_dir)
    gen_config = importlib.import_module("gen_config")
    algos = [0, 1, 2, 3, 7, 13, 19, 22]
    path = tmp_path / "cands.csv"
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=["cta_m", "cta_n", "cta_k", "stages", "raster", "cta_group", "runtime"])
        w.writeheader()
        for i, a in enumerate(algos):
            p = config.algo_params(a)
            w.writerow({"cta_m": p["BM"] * p["mt"], "cta_n": p["BN"], "cta_k": p["BK"], "stages": p["stages"],
                        "raster": p["raster"], "cta_group": 1 + p["cta2"], "runtime": 1.0 + i})
        w.writerow({"cta_m": 64, "cta_n": 64, "cta_k": 32, "stages": 3, "raster": 1, "cta_group": 1, "runtime": 0.5})
    assert gen_config.candidates_from_csv(str(path)) == algos      # the unknown row is skipped
    sys.modules.pop("gen_config", None)


def test_tuned_config_is_used_only_for_what_it_was_tuned_for(tmp_path):
    """A config searched for the counter-gated all-reduce at tp4 must not be picked up by a fused
    reduce-scatter (or another world size) of the same shape; files without the keys match."""
    import warnings
    from flashoverlap_b200.utils import config
    M, N, K = 512, 1024, 256
    path = config.config_path(M, N, K, "b200", tmp_path)
    config.save_solution(path, 128, 256, 0.1, 0, list(range(16)), [8, 8], 1, tp=4, comm_op="all_reduce", mode="gated")
    assert config.load_tuned(M, N, K, tp=4, comm_op="all_reduce", mode="gated", gpu="b200", directory=tmp_path)["cSeg"] == [8, 8]
    assert config.load_tuned(M, N, K, tp=4, comm_op="all_reduce", gpu="b200", directory=tmp_path) is not None
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        assert config.load_tuned(M, N, K, tp=4, comm_op="reduce_scatter", gpu="b200", directory=tmp_path) is None
        assert config.load_tuned(M, N, K, tp=8, comm_op="all_reduce", gpu="b200", directory=tmp_path) is None
        assert config.load_tuned(M, N, K, tp=4, comm_op="all_reduce", mode="fused", gpu="b200", directory=tmp_path) is None
        assert len(w) == 3 and "ignored" in str(w[0].message)
    # a stage-1 file (lists) is not a tuned config; a file without the optional keys matches any use
    config.save_stage1(path, [128], [256], [0.1], [0])
    assert config.load_tuned(M, N, K, tp=4, comm_op="all_reduce", gpu="b200", directory=tmp_path) is None
    config.save_solution(path, 128, 256, 0.1, 0, list(range(16)), [16], 1)
    assert config.load_tuned(M, N, K, tp=2, comm_op="reduce_scatter", mode="fused", gpu="b200", directory=tmp_path) is not None
    assert config.load_tuned(M + 128, N, K, gpu="b200", directory=tmp_path) is None
