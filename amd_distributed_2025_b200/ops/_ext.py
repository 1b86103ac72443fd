"""Build and load the native extension (C++ runtime + sm_100a kernels).

The reference compiles its kernels at import time on every rank with ``load_inline`` and
a hand-bumped module name to dodge stale caches (all2all/hipv8.py:241-252).  Here the
sources live in ``csrc/``; ``build()`` compiles them ahead of time into
``<package>/_C/b200_ext.so`` for ``sm_100a`` only, and ``load()`` imports that file
directly when a content hash of the sources matches, so ranks never race on a build and
a stale binary is never picked up.  Only when no matching binary exists does ``load()``
fall back to building (rank 0 first when a process group is up).
"""
from __future__ import annotations

import hashlib
import importlib.machinery
import importlib.util
import os
import sys
import threading
from typing import List

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC_DIR = os.path.join(_PKG_DIR, "csrc")
BUILD_DIR = os.path.join(_PKG_DIR, "_C")
EXT_NAME = "b200_ext"

CUDA_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
]

_lock = threading.Lock()
_module = None


def _source_files() -> List[str]:
    files = []
    for name in sorted(os.listdir(CSRC_DIR)):
        if name.endswith((".cu", ".cuh", ".cpp", ".h")):
            files.append(os.path.join(CSRC_DIR, name))
    return files


def source_hash() -> str:
    h = hashlib.sha256()
    for path in _source_files():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(CUDA_FLAGS).encode())
    return h.hexdigest()


def _so_path() -> str:
    return os.path.join(BUILD_DIR, EXT_NAME + ".so")


def _hash_path() -> str:
    return os.path.join(BUILD_DIR, EXT_NAME + ".hash")


def is_built() -> bool:
    try:
        with open(_hash_path(), "r", encoding="utf-8") as fh:
            return os.path.exists(_so_path()) and fh.read().strip() == source_hash()
    except OSError:
        return False


def build(verbose: bool = False) -> str:
    """Compile the extension in-tree for sm_100a; returns the path of the shared object."""
    import torch  # noqa: F401  (the extension links against libtorch)
    from torch.utils import cpp_extension

    os.makedirs(BUILD_DIR, exist_ok=True)
    sources = [f for f in _source_files() if f.endswith((".cu", ".cpp"))]
    cpp_extension.load(
        name=EXT_NAME,
        sources=sources,
        extra_include_paths=[CSRC_DIR],
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=CUDA_FLAGS,
        build_directory=BUILD_DIR,
        verbose=verbose,
        is_python_module=False,
    )
    with open(_hash_path(), "w", encoding="utf-8") as fh:
        fh.write(source_hash())
    return _so_path()


def _import_so():
    import torch  # noqa: F401

    loader = importlib.machinery.ExtensionFileLoader(EXT_NAME, _so_path())
    spec = importlib.util.spec_from_loader(EXT_NAME, loader)
    module = importlib.util.module_from_spec(spec)
    loader.exec_module(module)
    sys.modules[EXT_NAME] = module
    return module


def load(allow_build: bool = True):
    """Return the extension module, building it first if no up-to-date binary exists."""
    global _module
    with _lock:
        if _module is not None:
            return _module
        if not is_built():
            if not allow_build:
                raise RuntimeError(
                    f"native extension is not built (expected {_so_path()}); run "
                    "`python -c 'import __graft_entry__ as g; g.build()'` at the repository root"
                )
            _build_collectively()
        _module = _import_so()
        return _module


def _build_collectively() -> None:
    """One builder per node: rank 0 of the default group compiles, the others wait."""
    try:
        import torch.distributed as dist

        in_group = dist.is_available() and dist.is_initialized()
    except Exception:  # pragma: no cover
        in_group = False
    if not in_group:
        build()
        return
    import torch.distributed as dist

    if dist.get_rank() == 0:
        build()
    dist.barrier()
    if not is_built():
        raise RuntimeError("native extension build on rank 0 did not produce a matching binary")


def available() -> bool:
    """True when the binary is present (does not import it)."""
    return is_built()
