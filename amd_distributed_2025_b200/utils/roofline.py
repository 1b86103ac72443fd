"""Roofline arithmetic for the two fused paths.

Target time of a fused compute+collective kernel = the slower of FLOPs / measured GEMM
peak and bytes that must cross NVLink / measured per-direction link bandwidth.  The MoE
path moves bytes only.  Peaks come from ``MEASURED_PEAKS.json`` at the repository root
when present, else from the stated fallbacks.  The speed-of-light tables of the reference
(all2all/task.yml:38-44, gemm-rs/task.yml:47-54) are for other hardware and are carried
as data in ``configs/``, not used here.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NVLINK_GBS_PER_DIR = 770.0  # measured peer copy per direction on this class of machine; 900 nominal


def load_peaks(repo_root: Optional[str] = None) -> Dict[str, float]:
    root = repo_root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    peaks = dict(FALLBACK)
    peaks["source"] = "fallback"
    try:
        with open(path, "r", encoding="utf-8") as fh:
            data = json.load(fh)
        for k in FALLBACK:
            if k in data:
                peaks[k] = float(data[k])
        peaks["source"] = "measured"
    except (OSError, ValueError):
        pass
    peaks["nvlink_gbs_per_dir"] = NVLINK_GBS_PER_DIR
    return peaks


def gemm_rs_roofline_us(m: int, n: int, k_global: int, world_size: int, peaks: Dict[str, float],
                        sustained: bool = True) -> Dict[str, float]:
    """Per-rank FLOPs and NVLink bytes of a row-parallel GEMM + reduce-scatter."""
    flops = 2.0 * m * n * (k_global / world_size)
    tf = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    compute_us = flops / (tf * 1e12) * 1e6
    link_bytes = (world_size - 1) / world_size * m * n * 2.0  # bf16 partials leaving this rank
    link_us = link_bytes / (peaks["nvlink_gbs_per_dir"] * 1e9) * 1e6
    return {"flops": flops, "compute_us": compute_us, "link_bytes": link_bytes, "link_us": link_us,
            "roofline_us": max(compute_us, link_us)}


def moe_roofline_us(rows_out_remote: int, rows_in_remote: int, row_bytes: int, peaks: Dict[str, float]) -> Dict[str, float]:
    """Dispatch + combine each move every remote row once in each direction; the bound is
    the busier direction of the busier phase, counted twice (dispatch then combine)."""
    per_phase = max(rows_out_remote, rows_in_remote) * row_bytes
    us = per_phase / (peaks["nvlink_gbs_per_dir"] * 1e9) * 1e6
    return {"bytes_per_phase": per_phase, "roofline_us": 2.0 * us}
