"""Loader for the UNMODIFIED reference files, for comparison arms.

The reference is a directory of scripts, not a package (``all2all/reference.py`` and
``gemm-rs/reference.py`` both do ``from task import ...`` against the ``task.py`` beside
them), so each file is imported under a private name with its own directory first on
``sys.path``.  Nothing of the reference is re-implemented here: callers get its modules and
call its ``ref_kernel`` / ``generate_input`` / ``check_implementation`` as they are.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from typing import Optional

_REPO_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
DEFAULT_REF_DIR = os.path.join(_REPO_ROOT, "baseline", "_ref")


def reference_available(ref_dir: Optional[str] = None) -> bool:
    d = ref_dir or DEFAULT_REF_DIR
    return os.path.exists(os.path.join(d, "all2all", "reference.py")) and os.path.exists(
        os.path.join(d, "gemm-rs", "reference.py")
    )


def _load(name: str, path: str, extra_path: str):
    sys.modules.pop("task", None)
    sys.path.insert(0, extra_path)
    try:
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        sys.path.remove(extra_path)
        sys.modules.pop("task", None)
    return mod


def load_all2all(ref_dir: Optional[str] = None):
    """The reference's MoE module (MoEConfig, RankTestData, PyTorchAllToAll, ref_kernel, ...)."""
    d = os.path.join(ref_dir or DEFAULT_REF_DIR, "all2all")
    return _load("reference_all2all", os.path.join(d, "reference.py"), d)


def load_gemm_rs(ref_dir: Optional[str] = None):
    """The reference's GEMM + reduce-scatter module (generate_input, ref_kernel, ...)."""
    d = os.path.join(ref_dir or DEFAULT_REF_DIR, "gemm-rs")
    return _load("reference_gemm_rs", os.path.join(d, "reference.py"), d)


def moe_tuple(ref_module, cfg, data, rank: int, world_size: int):
    """This package's ``(cfg, data)`` handed over in the reference's own types."""
    rcfg = ref_module.MoEConfig(cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim, cfg.max_num_tokens,
                                cfg.in_dtype, cfg.out_dtype)
    rdata = object.__new__(ref_module.RankTestData)
    rdata.num_tokens, rdata.x, rdata.indices, rdata.weights = data.num_tokens, data.x, data.indices, data.weights
    return rcfg, rdata, rank, world_size
