"""Builds and loads the native extension (CUDA kernels + C++ runtime + torch bindings).

The shared object is built in-tree (``flashoverlap_b200/lib/``) for sm_100a only and is
loaded with ``torch.ops.load_library``; it registers
``torch.classes.flashoverlap_class.{OverlapImpl,BaselineImpl}`` and
``torch.ops.flashoverlap_op.*`` exactly where the reference's ``libst_pybinding.so`` puts them
(reference: src/CMakeLists.txt:28-38, README.md:68-70).  A content hash of the sources is kept
beside the library so that a stale build is detected without relying on file times.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import sysconfig
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_ROOT = _PKG.parent
_CSRC = _ROOT / "csrc"
_LIB_DIR = _PKG / "lib"
_LIB_NAME = "libflashoverlap_b200.so"
_EXT_NAME = "flashoverlap_b200_ext"

SOURCES = [
    "binding.cpp",
    "comm/nccl_utils.cpp",
    "comm/symmetric_heap.cpp",
    "runtime/overlap_impl.cpp",
    "runtime/baseline_impl.cpp",
    "runtime/loopback.cpp",
    "gemm/fo_gemm_launch.cu",
    "norm/fo_norm.cu",
    "flags/fo_wait.cu",
    "noalloc/fo_noalloc.cu",
]

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
]
# FLASHOVERLAP_DEBUG=1 in the environment of the build: the debug build, in which every overlap
# call validates the values of its index arrays on the host before launching (option "validate"
# defaults to 1).  The flag is part of the source hash, so switching it rebuilds.
DEBUG_BUILD = os.environ.get("FLASHOVERLAP_DEBUG", "0") == "1"
if DEBUG_BUILD:
    CUDA_FLAGS = CUDA_FLAGS + ["-DFO_DEBUG=1"]

_loaded = False


def lib_path() -> Path:
    return _LIB_DIR / _LIB_NAME


def _existing_sources() -> list[Path]:
    return [_CSRC / s for s in SOURCES if (_CSRC / s).exists()]


def source_hash() -> str:
    h = hashlib.sha256()
    files = sorted(p for p in _CSRC.rglob("*") if p.suffix in {".cu", ".cuh", ".h", ".cpp"})
    for p in files:
        h.update(str(p.relative_to(_CSRC)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(CUDA_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    stamp = _LIB_DIR / (_LIB_NAME + ".hash")
    return lib_path().exists() and stamp.exists() and stamp.read_text().strip() == source_hash()


def write_stamp() -> None:
    """Records the current source hash beside the library (the CMake build calls this)."""
    _LIB_DIR.mkdir(parents=True, exist_ok=True)
    (_LIB_DIR / (_LIB_NAME + ".hash")).write_text(source_hash() + "\n")


def _nccl_paths() -> tuple[str, str]:
    site = Path(sysconfig.get_paths()["purelib"])
    inc = site / "nvidia" / "nccl" / "include"
    lib = site / "nvidia" / "nccl" / "lib"
    if (inc / "nccl.h").exists() and (lib / "libnccl.so.2").exists():
        return str(inc), str(lib)
    return "/usr/include", "/usr/lib/x86_64-linux-gnu"


def _compile(verbose: bool = False) -> None:
    """Compiles the sources into the build directory (run in a child process by build())."""
    from torch.utils import cpp_extension

    build_dir = _ROOT / "build" / _EXT_NAME
    build_dir.mkdir(parents=True, exist_ok=True)
    nccl_inc, nccl_lib = _nccl_paths()
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    cpp_extension.load(
        name=_EXT_NAME,
        sources=[str(p) for p in _existing_sources()],
        extra_cflags=["-O2", "-std=c++17"] + (["-DFO_DEBUG=1"] if DEBUG_BUILD else []),
        extra_cuda_cflags=CUDA_FLAGS,
        extra_include_paths=[str(_CSRC), nccl_inc],
        extra_ldflags=[f"-L{nccl_lib}", "-l:libnccl.so.2", f"-Wl,-rpath,{nccl_lib}"],
        build_directory=str(build_dir),
        is_python_module=False,
        verbose=verbose,
    )


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every source for sm_100a and places the library in-tree.

    The compiler runs in a child process: ``cpp_extension.load`` maps the image it has just
    built (in the build directory) into the process that called it, and a process that later
    loads the in-tree copy as well would hold two images of the library - two sets of op
    registrations and two copies of every device symbol.  This process only ever maps
    ``lib_path()``, so a ``ctypes.CDLL(lib_path())`` gets the handle torch already holds."""
    if is_current() and not force:
        return lib_path()
    import subprocess
    import sys

    subprocess.run([sys.executable, "-c",
                    f"import sys; sys.path.insert(0, {str(_ROOT)!r}); "
                    f"from flashoverlap_b200 import _build; _build._compile({bool(verbose)!r})"],
                   check=True, cwd=str(_ROOT))
    built = _ROOT / "build" / _EXT_NAME / (_EXT_NAME + ".so")
    _LIB_DIR.mkdir(parents=True, exist_ok=True)
    shutil.copy2(built, lib_path())
    write_stamp()
    return lib_path()


def load(allow_build: bool = True) -> Path:
    """Loads the native library into this process (building it first if it is missing or stale)."""
    global _loaded
    if _loaded:
        return lib_path()
    import torch

    if not is_current():
        if not allow_build:
            raise RuntimeError(
                f"{lib_path()} is missing or stale; run `python -c 'import __graft_entry__ as g; g.build()'`")
        build()
    torch.ops.load_library(str(lib_path()))
    _loaded = True
    return lib_path()
