"""Evaluator: runs the task's test and benchmark shape lists on N ranks.

The reference names an evaluator (``eval.py``) and helpers that are not part of its tree
(all2all/task.yml:6-8, gemm-rs/task.yml:6-8); this module supplies that role.  For every
shape it builds the inputs on every rank (``generate_input``), calls the entry point under
test, checks the result with the task's tolerance against the communication-free oracle
and, in test mode on GPUs, also with the reference's own unmodified ``check_implementation``
(loaded from ``baseline/_ref``, run collectively on all ranks), and in benchmark mode times it with CUDA events, maximum over ranks, and ranks the run by
the geometric mean over shapes (all2all/task.yml:68, gemm-rs/task.yml:62).

Usage::

    python -m amd_distributed_2025_b200.harness.eval --task all2all --mode test --world-size 8
    torchrun --nproc-per-node 8 -m amd_distributed_2025_b200.harness.eval --task gemm_rs --mode benchmark

Without ``RANK`` in the environment the module spawns the ranks itself.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import sys
import traceback
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from .. import contract, oracle
from ..utils import timing


# --------------------------------------------------------------------------------------
# process plumbing
# --------------------------------------------------------------------------------------

def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def init_process_group(rank: int, world_size: int, backend: str, port: int, timeout_s: float = 600.0) -> None:
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    kwargs: Dict[str, Any] = {}
    if backend == "nccl":
        torch.cuda.set_device(rank % max(torch.cuda.device_count(), 1))
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(
        backend, rank=rank, world_size=world_size, timeout=datetime.timedelta(seconds=timeout_s), **kwargs
    )


def _worker(rank: int, world_size: int, backend: str, port: int, fn: Callable, args: tuple, result_dir: str) -> None:
    out: Dict[str, Any] = {"rank": rank, "ok": False}
    try:
        if backend == "gloo":
            # CPU ranks share the cores; leaving every rank at the default thread count makes
            # the intra-op pools fight each other
            torch.set_num_threads(max(1, (os.cpu_count() or world_size) // world_size))
        init_process_group(rank, world_size, backend, port)
        out["result"] = fn(rank, world_size, *args)
        out["ok"] = True
    except Exception:  # noqa: BLE001 - the parent re-raises with the traceback text
        out["error"] = traceback.format_exc()
        if backend == "nccl" and dist.is_initialized():
            # A GPU rank that failed still takes its workspaces down together with the others (they
            # reach their own teardown at the end of ``fn`` or after their bounded waits expire): no
            # rank may leave while a peer maps its slab, or while its memory is bound to an NVLink
            # multicast object that a peer can still read through.
            try:
                release_workspaces()
            except Exception:  # noqa: BLE001
                out["error"] += "\n(teardown after the failure also failed)\n" + traceback.format_exc()
    finally:
        with open(os.path.join(result_dir, f"rank{rank}.json"), "w", encoding="utf-8") as fh:
            json.dump(out, fh)
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # noqa: BLE001
                pass


def run_ranks(fn: Callable, world_size: int, backend: str = "gloo", args: tuple = (), timeout_s: float = 600.0) -> List[Any]:
    """Run ``fn(rank, world_size, *args)`` on ``world_size`` fresh processes and return the
    per-rank results (which must be JSON-serialisable).  Raises if any rank failed."""
    import tempfile

    port = free_port()
    with tempfile.TemporaryDirectory() as tmp:
        ctx = mp.get_context("spawn")
        procs = [
            ctx.Process(target=_worker, args=(r, world_size, backend, port, fn, args, tmp)) for r in range(world_size)
        ]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout_s)
        hung = [p for p in procs if p.is_alive()]
        for p in hung:
            p.kill()
        results = []
        for r in range(world_size):
            path = os.path.join(tmp, f"rank{r}.json")
            if not os.path.exists(path):
                raise RuntimeError(f"rank {r} produced no result (exit code {procs[r].exitcode}, hung={procs[r] in hung})")
            with open(path, "r", encoding="utf-8") as fh:
                results.append(json.load(fh))
    errors = [f"rank {r['rank']}:\n{r['error']}" for r in results if not r["ok"]]
    if errors:
        raise RuntimeError("\n".join(errors))
    return [r["result"] for r in results]


# --------------------------------------------------------------------------------------
# per-task evaluation
# --------------------------------------------------------------------------------------

def _device_for(rank: int) -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def moe_rank_data(spec: Dict[str, Any], rank: int, world_size: int, device: torch.device):
    """Input tuple of one rank.  Shapes from the task lists use the reference generator;
    shapes that fix ``tokens_per_rank`` use the benchmark factory."""
    if "tokens_per_rank" not in spec:
        return contract.generate_moe_input(
            spec["num_experts"], spec["experts_per_token"], spec["hidden_dim"], spec["max_num_tokens"],
            spec["seed"], rank, world_size, device=device,
        )
    return contract.make_moe_inputs(
        spec["num_experts"], spec["experts_per_token"], spec["hidden_dim"],
        spec.get("max_num_tokens", spec["tokens_per_rank"]),
        spec["seed"], rank, world_size, device=device,
        dtype=getattr(torch, spec.get("dtype", "float16")),
        fixed_num_tokens=spec["tokens_per_rank"],
        routing=spec.get("routing", "uniform"), weights=spec.get("weights", "rand"),
        zipf_s=spec.get("zipf_s", 1.2),
    )


_REFERENCE_MODULES: Dict[str, Any] = {}


def _reference_module(task: str):
    from . import reference_arm

    if task not in _REFERENCE_MODULES:
        _REFERENCE_MODULES[task] = reference_arm.load_all2all() if task == "all2all" else reference_arm.load_gemm_rs()
    return _REFERENCE_MODULES[task]


def reference_arm_data(cfg, mine, rank: int, world_size: int):
    from . import reference_arm

    return reference_arm.moe_tuple(_reference_module("all2all"), cfg, mine, rank, world_size)


def _literal_check(task: str, data, out) -> tuple:
    """``check_implementation(data, out)`` of the unmodified reference file (collective)."""
    ok, msg = _reference_module(task).check_implementation(data, out)
    return bool(ok), str(msg)


def literal_check_possible(device: torch.device, world_size: int) -> bool:
    """The reference's checker runs its oracle over ``torch.distributed`` on ``cuda:{rank}``
    tensors, so it needs GPUs, an initialised process group and the reference files."""
    from . import reference_arm

    return (device.type == "cuda" and dist.is_available() and dist.is_initialized()
            and dist.get_world_size() == world_size and reference_arm.reference_available())


def eval_moe_shape(rank: int, world_size: int, spec: Dict[str, Any], impl: str, mode: str,
                   warmup: int = 3, iters: int = 10, literal_check: bool = False) -> Dict[str, Any]:
    from ..models import moe_all2all
    from ..parallel import baseline_nccl

    device = torch.device(spec["device"]) if "device" in spec else _device_for(rank)
    cfg, mine, _, _ = moe_rank_data(spec, rank, world_size, device)
    data = (cfg, mine, rank, world_size)
    if impl == "reference":
        from . import reference_arm

        ref = reference_arm.load_all2all()
        ref_data = reference_arm.moe_tuple(ref, cfg, mine, rank, world_size)
        fn = lambda: ref.ref_kernel(ref_data)  # noqa: E731
    else:
        fn = {
            "ours": lambda: moe_all2all.custom_kernel(data),
            "torch": lambda: baseline_nccl.moe_torch(data),
        }[impl]
    out = fn()
    expected = oracle.moe_expected_output(cfg, mine, world_size, emulate_reference_rounding=True)
    ok, msg = oracle.check_moe_output(out, expected)
    res: Dict[str, Any] = {"spec": spec, "ok": bool(ok), "msg": msg, "num_tokens": mine.num_tokens}
    if literal_check and impl != "reference":
        # The task's own acceptance test, unmodified: it re-runs the reference's collective
        # oracle on these inputs, so every rank calls it together (all2all/reference.py:275-283).
        lit_ok, lit_msg = _literal_check("all2all", reference_arm_data(cfg, mine, rank, world_size), out)
        res["literal_ok"] = bool(lit_ok)
        if not lit_ok:
            res["ok"], res["msg"] = False, "reference check_implementation: " + lit_msg[:300]
    if impl == "ours" and device.type == "cuda":
        layer = moe_all2all.get_layer(cfg, rank, world_size)
        try:
            layer.check(sync=True)
        except Exception as exc:  # noqa: BLE001
            res["ok"], res["msg"] = False, str(exc)
    if mode == "benchmark":
        _benchmark(fn, device, world_size, warmup, iters, res)
    return res


def _benchmark(fn, device: torch.device, world_size: int, warmup: int, iters: int, res: Dict[str, Any]) -> None:
    """CUDA events on a GPU; wall clock around barrier-aligned calls on CPU ranks.  Max over ranks."""
    barrier = dist.barrier if world_size > 1 else None
    if device.type == "cuda":
        times = timing.time_cuda(fn, warmup=warmup, iters=iters, flush=True, barrier=barrier)
    else:
        import time

        for _ in range(warmup):
            fn()
        times = []
        for _ in range(iters):
            if barrier is not None:
                barrier()
            t0 = time.perf_counter()
            fn()
            times.append((time.perf_counter() - t0) * 1e3)
    times = timing.max_over_ranks(times)
    res["time_us"] = timing.summarize(times)["mean_ms"] * 1e3
    res["median_us"] = timing.summarize(times)["median_ms"] * 1e3


def eval_gemm_rs_shape(rank: int, world_size: int, spec: Dict[str, Any], impl: str, mode: str,
                       warmup: int = 3, iters: int = 10, literal_check: bool = False) -> Dict[str, Any]:
    from ..models import gemm_rs
    from ..parallel import baseline_nccl

    device = _device_for(rank)
    dist_kind = spec.get("dist", "reference")
    everyone = [
        contract.make_gemm_rs_inputs(r, world_size, spec["m"], spec["n"], spec["k"], spec["has_bias"], spec["seed"],
                                     device=device, dist=dist_kind)
        for r in range(world_size)
    ]
    data = everyone[rank]
    if impl == "reference":
        from . import reference_arm

        ref = reference_arm.load_gemm_rs()
        fn = lambda: ref.ref_kernel(data)  # noqa: E731
    else:
        fn = {
            "ours": lambda: gemm_rs.custom_kernel(data),
            "torch": lambda: baseline_nccl.gemm_rs_torch(data),
        }[impl]
    out = fn()
    a_all, w_all = [d[0] for d in everyone], [d[1] for d in everyone]
    truth = oracle.gemm_rs_truth(a_all, w_all, data[2], rank, dtype=torch.float32 if device.type == "cuda" else torch.float64)
    # Task tolerance against the result with the same rounding points (bf16 partials, as the
    # reference's matmul output has), plus a strict relative error against the un-rounded sum.
    ok, msg = oracle.check_gemm_rs_output(out, oracle.gemm_rs_fused_rounding(a_all, w_all, data[2], rank))
    rel = oracle.relative_error(out, truth)
    res: Dict[str, Any] = {"spec": spec, "ok": bool(ok and rel < 1e-2), "msg": msg, "rel_err": rel}
    if literal_check and impl != "reference" and dist_kind == "reference":
        # gemm-rs/reference.py:63-71, unmodified and collective; meaningful as an acceptance
        # gate only with the task's own operand distribution (see oracle.outlier_fraction)
        lit_ok, lit_msg = _literal_check("gemm_rs", data, out)
        res["literal_ok"] = bool(lit_ok)
        if not lit_ok:
            res["ok"], res["msg"] = False, "reference check_implementation: " + lit_msg[:300]
    if mode == "benchmark":
        _benchmark(fn, device, world_size, warmup, iters, res)
    return res


def run_task(rank: int, world_size: int, task: str, mode: str, impl: str, warmup: int, iters: int) -> List[Dict[str, Any]]:
    if task == "headline_cpu":
        # the fp32 two-rank CPU configuration of configs/headline.yml (device: cpu)
        specs = [dict(c) for c in contract.load_task("headline")["moe"] if c.get("device") == "cpu"]
        for c in specs:
            c["max_num_tokens"] = c["tokens_per_rank"]
        results = [eval_moe_shape(rank, world_size, c, impl, mode, warmup, iters) for c in specs]
        release_workspaces()
        return results
    specs = contract.task_specs(task, "tests" if mode == "test" else "benchmarks")
    literal = mode == "test" and impl == "ours" and literal_check_possible(_device_for(rank), world_size)
    results = []
    for spec in specs:
        spec = dict(spec)
        spec.pop("world_size", None)  # the list is written for 8 ranks; run on what we have
        if task == "all2all":
            if spec["num_experts"] % world_size:
                continue
            results.append(eval_moe_shape(rank, world_size, spec, impl, mode, warmup, iters, literal))
        else:
            if spec["m"] % world_size or spec["k"] % world_size:
                continue
            results.append(eval_gemm_rs_shape(rank, world_size, spec, impl, mode, warmup, iters, literal))
    release_workspaces()
    return results


def release_workspaces() -> None:
    """Collective, orderly teardown of every cached symmetric workspace of this process."""
    from ..models import gemm_rs, host_ops, moe_all2all

    if torch.cuda.is_available():
        torch.cuda.synchronize()
    moe_all2all.release_layers()
    gemm_rs.release_ops()
    host_ops.release()  # every rank holds its own mappings of the shared-memory slabs: no meeting needed


def summarize_results(results: List[Dict[str, Any]]) -> Dict[str, Any]:
    passed = sum(1 for r in results if r["ok"])
    out: Dict[str, Any] = {"shapes": len(results), "passed": passed}
    times = [r["time_us"] for r in results if "time_us" in r]
    if times:
        out["geomean_us"] = timing.geomean(times)
    return out


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--task", choices=["all2all", "gemm_rs", "headline_cpu"], required=True)
    ap.add_argument("--mode", choices=["test", "benchmark"], default="test")
    ap.add_argument("--impl", choices=["ours", "torch", "reference"], default="ours",
                    help="ours = this package; torch = vectorised torch.distributed restatement; "
                         "reference = the unmodified reference files under baseline/_ref")
    ap.add_argument("--world-size", type=int, default=None)
    ap.add_argument("--backend", default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None, help="write per-shape results to this file (rank 0)")
    args = ap.parse_args(argv)

    backend = args.backend or ("nccl" if torch.cuda.is_available() else "gloo")
    if args.task == "headline_cpu":
        backend = "gloo"
        args.world_size = args.world_size or 2
    if "RANK" in os.environ:
        rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist.init_process_group(backend)
        results = run_task(rank, ws, args.task, args.mode, args.impl, args.warmup, args.iters)
        dist.barrier()
        dist.destroy_process_group()
        per_rank = [results]
        if rank != 0:
            return 0
    else:
        ws = args.world_size or (torch.cuda.device_count() if torch.cuda.is_available() else 2)
        per_rank = run_ranks(run_task, ws, backend, (args.task, args.mode, args.impl, args.warmup, args.iters), 3600.0)
    results = per_rank[0]
    for i, r in enumerate(results):
        r["ok"] = all(pr[i]["ok"] for pr in per_rank)
        line = {k: v for k, v in r.items() if k != "msg" or v}
        print(json.dumps(line))
    summary = summarize_results(results)
    summary["literal_checker"] = sum(1 for r in results if r.get("literal_ok")) if any("literal_ok" in r for r in results) else None
    print(json.dumps({"task": args.task, "mode": args.mode, "impl": args.impl, "world_size": ws, **summary}))
    if args.json:
        with open(args.json, "w", encoding="utf-8") as fh:
            json.dump({"results": results, "summary": summary}, fh, indent=1)
    return 0 if summary["passed"] == summary["shapes"] else 1


if __name__ == "__main__":
    sys.exit(main())
