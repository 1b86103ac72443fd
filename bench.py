#!/usr/bin/env python
"""Headline benchmark: MoE dispatch+combine and GEMM + reduce-scatter latency.

One *step* runs each headline configuration once (configs/headline.yml):

  moe_decode           256 experts, top-8, hidden 7168, 128 tokens/rank, bf16, uniform routing
  moe_prefill_zipf     64 experts, top-6, hidden 4096, 4096 tokens/rank, bf16, Zipf(1.2) routing
  gemm_rs_large        M=N=8192, K=28672 split over the ranks, bias
  gemm_rs_sweep_m2048  M=2048, N=5120, K=12800 split over the ranks, bias
  gemm_rs_sweep_m256   M=256,  N=5120, K=12800 split over the ranks, bias

Every configuration is timed on the device with CUDA events (L2 flushed and all ranks
aligned by a barrier before each call), the maximum over ranks is taken per call, and
``value`` is the geometric mean over the configurations of the mean call time in
microseconds -- the ranking rule of the reference tasks (all2all/task.yml:68,
gemm-rs/task.yml:62).  ``e2e`` repeats the measurement through the public
``custom_kernel`` entry points with, inside the timed region of every call, the copy of
that call's inputs from pinned host memory to the device and the copy of its result back.

``--impl reference`` runs the unmodified reference files found under ``baseline/_ref``
(``ref_kernel`` of all2all/reference.py and gemm-rs/reference.py: torch.distributed over
NCCL plus the library GEMM) on the same inputs.

Launch: ``python bench.py`` (one GPU) or
``python -m torch.distributed.run --nproc-per-node N bench.py --gpus N``.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import statistics
import sys
import time
from typing import Any, Callable, Dict, List, Tuple

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from amd_distributed_2025_b200 import contract, oracle  # noqa: E402
from amd_distributed_2025_b200.harness import reference_arm  # noqa: E402
from amd_distributed_2025_b200.utils import timing  # noqa: E402
from amd_distributed_2025_b200.utils.clocks import ClockSampler  # noqa: E402

METRIC = "dispatch+combine us, GEMM-RS us (max over ranks), geomean over headline configs"
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
REF_MEASURED = os.path.join(ROOT, "baseline", "reference_measured.json")
# how a configuration grows with the number of GPUs: MoE keeps the tokens per rank (weak),
# GEMM-RS keeps the global problem and splits K (strong)
SCALING = {"moe": "weak", "gemm_rs": "strong"}


def stored_reference_value(n_gpus: int):
    """Geomean of the reference arm on this benchmark at ``n_gpus`` from an earlier run on the
    same kind of machine (baseline/reference_measured.json), or None."""
    try:
        with open(REF_MEASURED, "r", encoding="utf-8") as fh:
            return float(json.load(fh)["per_n"][str(n_gpus)]["value_us"])
    except (OSError, KeyError, ValueError):
        return None


def verify_output(item, y: torch.Tensor, rank: int, ws: int, device: torch.device) -> bool:
    """Compare a configuration's last result with the communication-free oracle (outside every
    timed region).  MoE: the task's tolerance against the expected combine; GEMM-RS: relative
    error against the un-rounded fp32 sum over all ranks' operands (the task tolerance is vacuous
    or noise-dominated for these operand distributions, see oracle.outlier_fraction)."""
    if item["kind"] == "moe":
        # against the exact weighted sum (fp64, one rounding): with bf16 the reference's own
        # per-add rounding strays further from it than the task tolerance allows
        want = oracle.moe_expected_output(item["cfg"], item["data"], ws)
        ok, _ = oracle.check_moe_output(y, want)
        return bool(ok)
    c = item["spec"]
    rows = c["m"] // ws
    acc = torch.zeros(rows, c["n"], dtype=torch.float32, device=device)
    for r in range(ws):  # regenerate the peers' operands here instead of moving them between GPUs
        a, w, _ = contract.make_gemm_rs_inputs(r, ws, c["m"], c["n"], c["k"], c["has_bias"], c["seed"], device=device)
        acc += a[rank * rows:(rank + 1) * rows].float() @ w.float().T
        del a, w
    if item["bias"] is not None:
        acc += ws * item["bias"].float()
    return oracle.relative_error(y, acc) < 5e-3


# --------------------------------------------------------------------------------------
# configurations and inputs
# --------------------------------------------------------------------------------------
def headline_configs() -> Tuple[List[Dict[str, Any]], List[Dict[str, Any]]]:
    cfg = contract.load_task("headline")
    moe = [c for c in cfg["moe"] if c.get("device", "cuda") != "cpu"]
    return moe, list(cfg["gemm_rs"])


def build_inputs(rank: int, ws: int, device: torch.device):
    """Device-resident inputs of every configuration plus pinned host copies for e2e."""
    moe_cfgs, gemm_cfgs = headline_configs()
    items = []
    for c in moe_cfgs:
        cfg, data, _, _ = contract.make_moe_inputs(
            c["num_experts"], c["experts_per_token"], c["hidden_dim"], c["tokens_per_rank"], c["seed"], rank, ws,
            device=device, dtype=getattr(torch, c["dtype"]), fixed_num_tokens=c["tokens_per_rank"],
            routing=c["routing"], weights=c["weights"], zipf_s=c.get("zipf_s", 1.2),
        )
        host = {k: getattr(data, k).cpu().pin_memory() for k in ("x", "indices", "weights")}
        items.append({"kind": "moe", "name": c["name"], "cfg": cfg, "data": data, "host": host, "spec": c})
    for c in gemm_cfgs:
        if c["m"] % ws or c["k"] % ws:
            continue
        a, w, bias = contract.make_gemm_rs_inputs(rank, ws, c["m"], c["n"], c["k"], c["has_bias"], c["seed"], device=device)
        items.append({"kind": "gemm_rs", "name": c["name"], "a": a, "w": w, "bias": bias,
                      "host": {"a": a.cpu().pin_memory()}, "spec": c})
    return items


# --------------------------------------------------------------------------------------
# implementations
# --------------------------------------------------------------------------------------
class Ours:
    name = "ours"
    def __init__(self, rank: int, ws: int):
        from amd_distributed_2025_b200.models import gemm_rs, moe_all2all

        # "dedup": dispatch (with the expert op) + combine; "direct": dispatch + expert scale + combine;
        # the fused GEMM-RS is one launch
        self.kernels_per_call = {"moe": 2 if moe_all2all.default_mode() == "dedup" else 3, "gemm_rs": 1}

        self.rank, self.ws = rank, ws
        self.moe, self.gemm = moe_all2all, gemm_rs

    def call(self, item) -> torch.Tensor:
        if item["kind"] == "moe":
            return self.moe.custom_kernel((item["cfg"], item["data"], self.rank, self.ws))
        return self.gemm.custom_kernel((item["a"], item["w"], item["bias"]))

    def call_with(self, item, dev_inputs) -> torch.Tensor:
        if item["kind"] == "moe":
            d = object.__new__(contract.RankTestData)
            d.num_tokens = item["data"].num_tokens
            d.x, d.indices, d.weights = dev_inputs["x"], dev_inputs["indices"], dev_inputs["weights"]
            return self.moe.custom_kernel((item["cfg"], d, self.rank, self.ws))
        return self.gemm.custom_kernel((dev_inputs["a"], item["w"], item["bias"]))

    def check(self) -> None:
        for layer in self.moe._LAYERS.values():
            layer.check(sync=True)
        for op in self.gemm._OPS.values():
            op.check(sync=True)

    def release(self) -> None:
        """Collective, orderly teardown of the symmetric workspaces (no slab is freed while a
        peer still maps it)."""
        torch.cuda.synchronize()
        self.moe.release_layers()
        self.gemm.release_ops()


class Reference:
    """The reference's own code, unmodified, imported from baseline/_ref."""

    name = "reference"
    kernels_per_call = {"moe": 0, "gemm_rs": 0}

    def __init__(self, rank: int, ws: int):
        self.rank, self.ws = rank, ws
        self.a2a = reference_arm.load_all2all(REF_DIR)
        self.grs = reference_arm.load_gemm_rs(REF_DIR)

    def _moe_tuple(self, item, x, indices, weights):
        d = object.__new__(contract.RankTestData)
        d.num_tokens, d.x, d.indices, d.weights = item["data"].num_tokens, x, indices, weights
        return reference_arm.moe_tuple(self.a2a, item["cfg"], d, self.rank, self.ws)

    def call(self, item) -> torch.Tensor:
        if item["kind"] == "moe":
            d = item["data"]
            return self.a2a.ref_kernel(self._moe_tuple(item, d.x, d.indices, d.weights))
        return self.grs.ref_kernel((item["a"], item["w"], item["bias"]))

    def call_with(self, item, dev_inputs) -> torch.Tensor:
        if item["kind"] == "moe":
            return self.a2a.ref_kernel(self._moe_tuple(item, dev_inputs["x"], dev_inputs["indices"], dev_inputs["weights"]))
        return self.grs.ref_kernel((dev_inputs["a"], item["w"], item["bias"]))

    def check(self) -> None:
        pass

    def release(self) -> None:
        pass


# --------------------------------------------------------------------------------------
# measurement
# --------------------------------------------------------------------------------------
def _barrier(ws: int) -> None:
    if ws > 1:
        dist.barrier()


def timed_call(fn: Callable[[], Any], ws: int) -> float:
    timing.flush_l2()
    torch.cuda.synchronize()
    _barrier(ws)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop)


def e2e_call(impl, item, out_host: Dict[str, torch.Tensor]) -> Callable[[], None]:
    def run():
        dev = {k: v.to("cuda", non_blocking=True) for k, v in item["host"].items()}
        y = impl.call_with(item, dev)
        buf = out_host.get(item["name"])
        if buf is None or buf.shape != y.shape:
            buf = torch.empty(y.shape, dtype=y.dtype).pin_memory()
            out_host[item["name"]] = buf
        buf.copy_(y, non_blocking=True)
    return run


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--only", default=None, help="comma-separated configuration names (debugging aid)")
    args = ap.parse_args()
    warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if ws != args.gpus:
        if rank == 0:
            print(json.dumps({"error": f"--gpus {args.gpus} but WORLD_SIZE={ws}; launch with torch.distributed.run"}))
        return 2
    if args.impl == "reference" and not reference_arm.reference_available(REF_DIR):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no copy of the reference files"}))
        return 0

    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"error": "no CUDA device: the headline benchmark runs on B200 GPUs only"}))
        return 2
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if ws > 1 or args.impl == "reference":
        if "MASTER_ADDR" not in os.environ:
            os.environ["MASTER_ADDR"] = "127.0.0.1"
            with socket.socket() as s:
                s.bind(("127.0.0.1", 0))
                os.environ["MASTER_PORT"] = str(s.getsockname()[1])
        dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=device)

    impl = Ours(rank, ws) if args.impl == "ours" else Reference(rank, ws)
    items = build_inputs(rank, ws, device)
    if args.only:
        keep = set(args.only.split(","))
        items = [it for it in items if it["name"] in keep]
    out_host: Dict[str, torch.Tensor] = {}

    # ---- warm-up (also creates the symmetric workspaces, which is collective) -----------
    for _ in range(warmup):
        for it in items:
            impl.call(it)
    for it in items:
        e2e_call(impl, it, out_host)()
    torch.cuda.synchronize()
    impl.check()
    _barrier(ws)

    # ---- device-timed region: exactly `steps` steps ---------------------------------------
    sampler = ClockSampler(local_rank, uuid=str(torch.cuda.get_device_properties(local_rank).uuid))
    if rank == 0:
        sampler.start()
    torch.cuda.synchronize()
    _barrier(ws)
    wall0 = time.perf_counter()
    dev_ms: Dict[str, List[float]] = {it["name"]: [] for it in items}
    for _ in range(args.steps):
        for it in items:
            dev_ms[it["name"]].append(timed_call(lambda it=it: impl.call(it), ws))
    torch.cuda.synchronize()
    _barrier(ws)
    wall_dev = time.perf_counter() - wall0
    clocks = sampler.stop() if rank == 0 else {}

    # ---- end-to-end region ------------------------------------------------------------------
    e2e_ms: Dict[str, List[float]] = {it["name"]: [] for it in items}
    for _ in range(args.steps):
        for it in items:
            e2e_ms[it["name"]].append(timed_call(e2e_call(impl, it, out_host), ws))
    torch.cuda.synchronize()
    impl.check()

    # ---- outputs against the oracle (untimed; every rank checks its own slice) ----------------
    checked: Dict[str, bool] = {}
    for it in items:
        y = impl.call(it)
        torch.cuda.synchronize()
        ok = verify_output(it, y, rank, ws, device)
        if ws > 1:
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = bool(flag.item())
        checked[it["name"]] = ok
        del y

    per_config = {}
    for it in items:
        name = it["name"]
        d = timing.max_over_ranks(dev_ms[name])
        e = timing.max_over_ranks(e2e_ms[name])
        per_config[name] = {
            "us": statistics.fmean(d) * 1e3,
            "median_us": statistics.median(d) * 1e3,
            "min_us": min(d) * 1e3,
            "e2e_us": statistics.fmean(e) * 1e3,
            "scaling": SCALING[it["kind"]],
            "checked": checked[name],
        }
    if rank == 0:
        value = timing.geomean([v["us"] for v in per_config.values()])
        e2e_value = timing.geomean([v["e2e_us"] for v in per_config.values()])
        h2d = sum(sum(t.numel() * t.element_size() for t in it["host"].values()) for it in items)
        d2h = sum(t.numel() * t.element_size() for t in out_host.values())
        launches = sum(impl.kernels_per_call[it["kind"]] for it in items) * args.steps
        aggregates = {}
        for kind, label in SCALING.items():
            names = [it["name"] for it in items if it["kind"] == kind]
            if names:
                aggregates[kind] = {"value": timing.geomean([per_config[nm]["us"] for nm in names]),
                                    "e2e": timing.geomean([per_config[nm]["e2e_us"] for nm in names]),
                                    "unit": "us", "scaling": label, "configs": names}
        ref_value = stored_reference_value(ws) if args.only is None else None
        line = {
            "metric": METRIC,
            "value": value,
            "unit": "us",
            "impl": args.impl,
            "n_gpus": ws,
            "steps": args.steps,
            "warmup": warmup,
            "ms_per_step": sum(v["us"] for v in per_config.values()) / 1e3,
            "higher_is_better": False,
            # the geomean mixes weak-scaled MoE and strong-scaled GEMM-RS configurations: read the
            # curve per configuration (per_config_us[*].scaling) or per family (aggregates)
            "scaling": "mixed",
            "vs_baseline": (value / ref_value) if ref_value else None,
            "baseline_source": "baseline/reference_measured.json (reference arm on B200, same N)" if ref_value else None,
            "checked": all(checked.values()),
            "dtype": "bf16",
            "data": "synthetic (seeded); random-init operands of the named shapes",
            "config": {
                "model": "MoE EP dispatch+combine (decode 256e/top8/h7168/128tok, prefill 64e/top6/h4096/4096tok Zipf1.2) "
                         "+ row-parallel GEMM-RS (8192x8192x28672, 2048x5120x12800, 256x5120x12800; bias)",
                "global_batch": "MoE: tokens per rank fixed (weak); GEMM-RS: global M,N,K fixed, K split over ranks (strong)",
                "seq_len": None,
                "parallelism": f"ep{ws}+tp{ws}",
                "l2": "flushed before every timed call (256 MiB write)",
                "timing": "CUDA events per call, max over ranks, mean over steps, geomean over configs",
            },
            "per_config_us": per_config,
            "aggregates": aggregates,
            "e2e": {"value": e2e_value, "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches,
            "clocks": clocks,
            "wall_s_timed_region": wall_dev,
        }
        print(json.dumps(line))
    impl.release()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


def _release_after_failure() -> None:
    """A rank that failed still takes its cached workspaces down together with the others before
    it exits (they fail too, at the latest when their bounded waits expire): no slab is freed
    while a peer maps it, no memory leaves an NVLink multicast object that a peer can still read."""
    try:
        from amd_distributed_2025_b200.models import gemm_rs, moe_all2all

        if torch.cuda.is_available():
            torch.cuda.synchronize()
        moe_all2all.release_layers()
        gemm_rs.release_ops()
    except Exception:  # noqa: BLE001 - the original failure is the one to report
        pass


if __name__ == "__main__":
    try:
        code = main()
    except Exception:
        _release_after_failure()
        raise
    sys.exit(code)
