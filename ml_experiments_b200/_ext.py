"""Builds (when stale) and loads the in-tree sm_100a extension that registers the ``torch.ops.b200`` operators.

The shared library is linked inside the package (``_build/b200_C.so``) so that it is found by
whoever imports the package from a copy of the source tree. A digest of the sources is stored beside the
library; the library is rebuilt only when that digest changes.
"""
from __future__ import annotations

import hashlib
import os
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_CSRC = _PKG / "csrc"
_BUILD = _PKG / "_build"
_NAME = "b200_C"
_lock = threading.Lock()
_loaded = False

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
]


def sources() -> list[Path]:
    out = [p for p in sorted(_CSRC.rglob("*")) if p.suffix in (".cu", ".cpp")]
    return out


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(_CSRC.rglob("*")):
        if p.suffix in (".cu", ".cpp", ".h", ".cuh"):
            h.update(str(p.relative_to(_CSRC)).encode())
            h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def lib_path() -> Path:
    return _BUILD / f"{_NAME}.so"


def is_current() -> bool:
    stamp = _BUILD / "sources.sha256"
    return lib_path().exists() and stamp.exists() and stamp.read_text().strip() == _digest()


def build(verbose: bool = False) -> Path:
    """Compile every CUDA/C++ source for sm_100a and link ``_build/b200_C.so`` (no GPU needed)."""
    from torch.utils import cpp_extension

    _BUILD.mkdir(exist_ok=True)
    if is_current():
        return lib_path()
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 8))
    cpp_extension.load(
        name=_NAME,
        sources=[str(p) for p in sources()],
        extra_cflags=["-O2", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS,
        extra_include_paths=[str(_CSRC)],
        build_directory=str(_BUILD),
        is_python_module=False,
        verbose=verbose,
    )
    (_BUILD / "sources.sha256").write_text(_digest())
    return lib_path()


def load() -> None:
    """Make ``torch.ops.b200.*`` available. Raises if the library cannot be built or loaded."""
    global _loaded
    if _loaded:
        return
    with _lock:
        if _loaded:
            return
        import torch

        if not is_current():
            build()
        torch.ops.load_library(str(lib_path()))
        _loaded = True


def available() -> bool:
    """True when a CUDA device is present (the operators only have CUDA implementations)."""
    import torch

    return torch.cuda.is_available()
