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
NVLINK_GBS_PER_DIR = 700.0  # measured: a kernel's peer stores, per direction (harness/link_probe.py); 900 nominal


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


# --------------------------------------------------------------------------------------
# report for a bench.py line
# --------------------------------------------------------------------------------------

def _moe_remote_rows(spec: Dict, world_size: int) -> Dict[str, int]:
    """Rows leaving / entering the busiest rank in one direction, from a seeded CPU draw of the
    same routing distribution (the realised count matrix of a run differs only statistically).
    A token counts once per destination RANK, however many of its experts live there: that is
    what the default protocol sends (csrc/moe_dedup.cu)."""
    import torch

    from .. import contract

    if world_size == 1:
        return {"out": 0, "in": 0}
    e_local = spec["num_experts"] // world_size
    sent = [[0] * world_size for _ in range(world_size)]
    for r in range(world_size):
        _, d, _, _ = contract.make_moe_inputs(
            spec["num_experts"], spec["experts_per_token"], 8, spec["tokens_per_rank"], spec.get("seed", 0), r, world_size,
            device="cpu", dtype=torch.float32, fixed_num_tokens=spec["tokens_per_rank"],
            routing=spec.get("routing", "uniform"), weights="rand", zipf_s=spec.get("zipf_s", 1.2),
        )
        owner = d.indices.to(torch.int64) // e_local  # [T, k]
        hit = torch.zeros(owner.shape[0], world_size, dtype=torch.bool)
        hit.scatter_(1, owner, True)
        sent[r] = hit.sum(0).tolist()
    out_rows = max(sum(sent[r][o] for o in range(world_size) if o != r) for r in range(world_size))
    in_rows = max(sum(sent[r][o] for r in range(world_size) if r != o) for o in range(world_size))
    return {"out": out_rows, "in": in_rows}


def report(bench_line: Dict, peaks: Optional[Dict[str, float]] = None) -> Dict[str, Dict[str, float]]:
    """Roofline and achieved fraction for every configuration of a ``bench.py`` JSON line."""
    from .. import contract

    peaks = peaks or load_peaks()
    ws = int(bench_line["n_gpus"])
    cfg = contract.load_task("headline")
    specs = {c["name"]: ("moe", c) for c in cfg["moe"]}
    specs.update({c["name"]: ("gemm_rs", c) for c in cfg["gemm_rs"]})
    out: Dict[str, Dict[str, float]] = {}
    for name, measured in bench_line.get("per_config_us", {}).items():
        kind, spec = specs[name]
        if kind == "gemm_rs":
            r = gemm_rs_roofline_us(spec["m"], spec["n"], spec["k"], ws, peaks)
            roof = r["roofline_us"]
        else:
            rows = _moe_remote_rows(spec, ws)
            row_bytes = spec["hidden_dim"] * 2
            link = moe_roofline_us(rows["out"], rows["in"], row_bytes, peaks)["roofline_us"]
            # local floor: per entry one write each of expert_x and expert_y and one read of expert_y,
            # per token one read of x and one write of the result
            local_bytes = (3.0 * spec["experts_per_token"] + 2.0) * spec["tokens_per_rank"] * row_bytes
            roof = max(link, local_bytes / (peaks["hbm_gbs"] * 1e9) * 1e6)
        out[name] = {"measured_us": measured["us"], "roofline_us": roof, "fraction_of_roofline": roof / measured["us"]}
    return out


def main(argv=None) -> int:
    import argparse
    import sys

    ap = argparse.ArgumentParser(description="Roofline fractions for a bench.py JSON line (file or stdin).")
    ap.add_argument("bench_json", nargs="?", default="-")
    args = ap.parse_args(argv)
    text = sys.stdin.read() if args.bench_json == "-" else open(args.bench_json, "r", encoding="utf-8").read()
    line = next(json.loads(l) for l in text.splitlines() if l.strip().startswith("{") and "per_config_us" in l)
    peaks = load_peaks()
    print(f"peaks ({peaks['source']}): HBM {peaks['hbm_gbs']:.0f} GB/s, bf16 sustained {peaks['bf16_tflops_sustained']:.0f} TFLOP/s, "
          f"NVLink {peaks['nvlink_gbs_per_dir']:.0f} GB/s per direction")
    for name, r in report(line, peaks).items():
        print(f"{name:24s} measured {r['measured_us']:10.1f} us   roofline {r['roofline_us']:9.1f} us   "
              f"achieved {r['fraction_of_roofline']:.2f} of roofline")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
