"""flashoverlap_b200: GEMM + collective overlap for tensor-parallel layers on B200 (sm_100a).

Public surface, mirroring the reference project (README.md:60-160 there):

* ``torch.classes.flashoverlap_class.OverlapImpl`` / ``BaselineImpl`` and
  ``torch.ops.flashoverlap_op.*`` once :func:`load_library` has run;
* ``flashoverlap_b200.models``: ``RowParallelLayer``, ``OverlapRowParallelLayer``, ``RMSNorm``,
  ``ReorderRMSNorm`` and a Llama-style tensor-parallel decoder layer;
* ``flashoverlap_b200.utils``: tile orders / layouts (``layout``) and the JSON config format
  (``config``);
* ``flashoverlap_b200.parallel``: process bootstrap helpers and the CPU functional models.
"""
from ._build import build as build_library, lib_path, load as load_library  # noqa: F401

__version__ = "0.1.0"
__all__ = ["build_library", "load_library", "lib_path", "__version__"]
