"""Reference arm of bench.py: runs the UNMODIFIED reference library (built from the read-only
reference tree into the git-ignored ``baseline/_ref``) through its own public API -
``torch.classes.flashoverlap_class.OverlapImpl.gemm_allreduce_overlap`` - on the benchmark shape.

The reference is fp16-only (src/overlap_impl.cu:222-227 casts every operand to ``at::Half``) with
fp16 accumulation; the shape, the timing protocol and the end-to-end harness are the ones the
product arm uses.  Its tuning inputs are produced the way its own scripts do it, in-process:
Algo by timing candidates (tune/profile_config.py:85-93), the hint by a monitor run
(tune/search.py:111-157), the wave grouping by timing a few partitions (tune/search.py:387-439).
Nothing of this repository's kernels or engine is on that path.
"""
from __future__ import annotations

import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
REF_LIB = os.path.join(REF_DIR, "lib", "libst_pybinding.so")


def unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        import bench
        print(json.dumps({"impl": "reference", "unavailable": why}), file=bench.REAL_STDOUT, flush=True)


def main(args) -> None:
    if not os.path.exists(REF_LIB):
        note = os.path.join(REF_DIR, "UNAVAILABLE.txt")
        why = open(note).read().strip().splitlines()[0] if os.path.exists(note) else \
            "reference library has not been built into baseline/_ref"
        unavailable(why)
        return
    from baseline import reference_run
    reference_run.run(args, REF_LIB)
