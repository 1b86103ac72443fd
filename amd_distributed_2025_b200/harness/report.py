"""Side-by-side benchmark report: every shape of a task's benchmark list on several arms.

The reference ranks a submission by the geometric mean of its times over the task's
benchmark shapes (all2all/task.yml:68, gemm-rs/task.yml:62) and quotes an analytic
speed-of-light per shape (all2all/task.yml:70-76, gemm-rs/task.yml:64-85); it ships no tool
that produces the comparison.  This one runs the evaluator (harness/eval.py) once per arm --
``ours``, ``torch`` (library collectives) and ``reference`` (the unmodified reference files,
when a copy is present) -- on the same ranks and inputs, and prints one markdown table per
task: time per shape and arm, the ratio to the first arm, the task's speed-of-light column,
and the geometric means.

    python -m amd_distributed_2025_b200.harness.report --tasks all2all,gemm_rs --arms ours,torch --world-size 8
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Any, Dict, List, Optional

import torch

from .. import contract
from ..utils import timing
from . import eval as evaluator


def _shape_key(task: str, spec: Dict[str, Any]) -> str:
    if task == "gemm_rs":
        return f"{spec['m']}, {spec['n']}, {spec['k']}, {'bias' if spec['has_bias'] else 'no bias'}"
    if "tokens_per_rank" in spec:
        return spec.get("name", "cpu")
    return f"{spec['num_experts']}, {spec['experts_per_token']}, {spec['hidden_dim']}, {spec['max_num_tokens']}"


def speed_of_light(task: str) -> Dict[str, float]:
    """The task's analytic lower bounds (microseconds, quoted for 8 x MI300X) keyed like the rows."""
    if task not in ("all2all", "gemm_rs"):
        return {}
    out = {}
    for s in contract.load_task(task).get("speed_of_light", []):
        spec = dict(s)
        spec.setdefault("has_bias", False)
        key = _shape_key(task, spec)
        out[key] = float(s["time_us"])
        if task == "gemm_rs":  # the table does not distinguish bias / no bias
            out[key.replace("no bias", "bias")] = float(s["time_us"])
    return out


def collect(task: str, arms: List[str], world_size: int, backend: str, warmup: int, iters: int,
            timeout_s: float = 3600.0) -> Dict[str, List[Dict[str, Any]]]:
    """``{arm: per-shape results of rank 0}``; every arm runs in fresh rank processes."""
    out = {}
    for arm in arms:
        per_rank = evaluator.run_ranks(evaluator.run_task, world_size, backend, (task, "benchmark", arm, warmup, iters),
                                       timeout_s)
        results = per_rank[0]
        for i, r in enumerate(results):
            r["ok"] = all(pr[i]["ok"] for pr in per_rank)
        out[arm] = results
    return out


def render(task: str, world_size: int, by_arm: Dict[str, List[Dict[str, Any]]]) -> str:
    arms = list(by_arm)
    base = arms[0]
    sol = speed_of_light(task)
    head = ["shape"] + [f"{a} us" for a in arms] + [f"{a} / {base}" for a in arms[1:]] + ["task speed of light us", "check"]
    lines = [f"### {task}, {world_size} ranks", "", "| " + " | ".join(head) + " |", "|" + "---|" * len(head)]
    n = len(by_arm[base])
    for i in range(n):
        key = _shape_key(task, by_arm[base][i]["spec"])
        t = [by_arm[a][i].get("time_us") for a in arms]
        row = [key] + [f"{v:.1f}" if v is not None else "-" for v in t]
        row += [f"{v / t[0]:.2f}x" if v is not None and t[0] else "-" for v in t[1:]]
        row.append(f"{sol[key]:.2f}" if key in sol else "-")
        row.append("passes" if all(by_arm[a][i]["ok"] for a in arms) else
                   "FAILS: " + ", ".join(a for a in arms if not by_arm[a][i]["ok"]))
        lines.append("| " + " | ".join(row) + " |")
    geo = []
    for a in arms:
        times = [r["time_us"] for r in by_arm[a] if "time_us" in r]
        geo.append(timing.geomean(times) if times else None)
    row = ["geometric mean"] + [f"**{g:.1f}**" if g is not None else "-" for g in geo]
    row += [f"{g / geo[0]:.2f}x" if g is not None and geo[0] else "-" for g in geo[1:]]
    row += ["-", ""]
    lines.append("| " + " | ".join(row) + " |")
    return "\n".join(lines) + "\n"


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--tasks", default="all2all,gemm_rs", help="comma-separated: all2all, gemm_rs, headline_cpu")
    ap.add_argument("--arms", default="ours,torch", help="comma-separated: ours, torch, reference; ratios are to the first")
    ap.add_argument("--world-size", type=int, default=None)
    ap.add_argument("--backend", default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default=None, help="also write the markdown here")
    ap.add_argument("--json", default=None, help="write the raw per-shape results here")
    args = ap.parse_args(argv)

    arms = [a for a in args.arms.split(",") if a]
    raw: Dict[str, Any] = {}
    text = []
    ok = True
    for task in [t for t in args.tasks.split(",") if t]:
        gpu = torch.cuda.is_available() and task != "headline_cpu"
        ws = args.world_size or (torch.cuda.device_count() if gpu else 2)
        backend = args.backend or ("nccl" if gpu else "gloo")
        by_arm = collect(task, arms, ws, backend, args.warmup, args.iters)
        raw[task] = {"world_size": ws, "arms": by_arm}
        ok &= all(r["ok"] for rs in by_arm.values() for r in rs)
        text.append(render(task, ws, by_arm))
    report = "\n".join(text)
    print(report)
    if args.out:
        with open(args.out, "w", encoding="utf-8") as fh:
            fh.write(report)
    if args.json:
        with open(args.json, "w", encoding="utf-8") as fh:
            json.dump(raw, fh, indent=1)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
