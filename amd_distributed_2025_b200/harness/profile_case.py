"""Run ONE small case of one kernel a few times on one GPU -- the workload to put under a
profiler (``ncu -k regex:<kernel> -c <n> python -m ...profile_case ...``) or to trace with
the kernels' own phase stamps.

The cases are sized for profiling: operands a little larger than the 126 MB L2 so DRAM
counters mean something, a few hundred MB on the device at most, a handful of launches.
The reference has no profiling hooks (timing is left to an evaluator outside its tree,
all2all/task.yml:6-8).

Examples::

    python -m amd_distributed_2025_b200.harness.profile_case --kernel gemm_rs --m 8192 --n 4096 --k 4096
    python -m amd_distributed_2025_b200.harness.profile_case --kernel gemm_rs --m 2048 --n 2048 --k 2048 --staged
    python -m amd_distributed_2025_b200.harness.profile_case --kernel moe --experts 256 --topk 8 --hidden 7168 --tokens 128
    python -m amd_distributed_2025_b200.harness.profile_case --kernel fp8_gemm --m 4096 --n 4096 --k 4096
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m amd_distributed_2025_b200.harness.profile_case --kernel gemm_rs --gemm-m 8192 --gemm-n 8192 --gemm-k 28672 --trace

Under ``torch.distributed.run`` the gemm_rs case runs on all ranks (``--k`` is the global K, split
evenly) and every rank prints its own line; ``--trace`` adds the in-kernel phase stamps.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from .. import contract, oracle
from ..utils import timing


def _host_time_us(fn, ws: int, iters: int = 20) -> float:
    """Median wall time the host spends inside the call (the GPU is idle when it starts): the
    part of a short call's event time that is Python, argument conversion and launch."""
    import statistics
    import time

    samples = []
    for _ in range(iters):
        torch.cuda.synchronize()
        if ws > 1:
            dist.barrier()
        t0 = time.perf_counter()
        fn()
        samples.append((time.perf_counter() - t0) * 1e6)
        torch.cuda.synchronize()
    return round(statistics.median(samples), 1)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernel", choices=["gemm_rs", "moe", "fp8_gemm"], required=True)
    # the long spellings are for torch.distributed.run, whose own parser trips over "--m"
    ap.add_argument("--m", "--gemm-m", dest="m", type=int, default=8192)
    ap.add_argument("--n", "--gemm-n", dest="n", type=int, default=4096)
    ap.add_argument("--k", "--gemm-k", dest="k", type=int, default=4096)
    ap.add_argument("--staged", action="store_true", help="gemm_rs: run the multi-rank staging/reduction path on one GPU")
    ap.add_argument("--trace", action="store_true", help="print the in-kernel phase stamps of the last launch")
    ap.add_argument("--mode", default=None, help="moe: protocol, dedup (default) or direct")
    ap.add_argument("--routing", default="uniform", help="moe: uniform or zipf")
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--rs-mode", default=None, help="gemm_rs on several ranks: p2p (default) or nvls")
    ap.add_argument("--few-launches", action="store_true",
                    help="for a run under a profiler: one warm-up call, --iters timed calls, no host-time loop")
    ap.add_argument("--fuse-own", choices=["auto", "on", "off"], default="auto",
                    help="gemm_rs on several ranks: finish own tiles in their epilogue, or in a pass after the GEMM tiles")
    args = ap.parse_args(argv)
    if args.rs_mode:
        os.environ["B200_RS_MODE"] = args.rs_mode
    rank, ws = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if ws > 1:
        if args.kernel == "fp8_gemm":
            raise SystemExit("the fp8_gemm case runs on one rank")
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    out = {"kernel": args.kernel, "rank": rank, "world_size": ws}
    if args.kernel == "gemm_rs":
        from ..models import gemm_rs

        k_local = args.k // ws
        a, w, bias = contract.make_gemm_rs_inputs(rank, ws, args.m, args.n, args.k, True, 1, device="cuda")
        op = gemm_rs.get_op(args.m, args.n, k_local)
        op.force_staged = args.staged
        op.fuse_own = {"auto": None, "on": True, "off": False}[args.fuse_own]
        if args.trace:
            op.enable_trace(True)
        times = timing.time_cuda(lambda: op(a, w, bias), warmup=3 if ws > 1 else 1, iters=args.iters,
                                 barrier=dist.barrier if ws > 1 else None)
        op.check()
        if not args.few_launches:
            out["host_us"] = _host_time_us(lambda: gemm_rs.custom_kernel((a, w, bias)), ws)
        if args.trace:
            op.trace.zero_()
        y = op(a, w, bias)
        torch.cuda.synchronize()
        out.update(shape=[args.m, args.n, args.k], plan=dict(op.plan(args.m, args.n, k_local)), rs_mode=op.rs_mode,
                   us=[t * 1e3 for t in times],
                   tflops_per_gpu=2.0 * args.m * args.n * k_local / min(times) / 1e9)
        if ws == 1:
            out["rel_err"] = oracle.relative_error(y, a.float() @ w.float().T + bias.float())
        if args.trace:
            tr = op.trace.cpu()
            tr = tr[tr[:, 0] > 0]
            t0 = tr[:, 0].min()
            fused = op.fuse_own if op.fuse_own is not None else ws <= 4
            names = {1: "pipeline_ready", 2: "gemm_tiles_done", 3: "exit"}
            names.update({4: "first_own_tile", 5: "peers_rows_arrived", 6: "last_own_tile_stored"} if fused else
                         {5: "first_unit_complete_after_gemm", 6: "last_unit_reduced"})
            stamps = {}
            for col, name in names.items():
                c = tr[:, col]
                c = c[c > 0]
                if len(c):
                    rel = (c - t0).float() / 1e3
                    stamps[name] = [round(float(rel.min()), 1), round(float(rel.median()), 1), round(float(rel.max()), 1)]
            out["trace_us_min_median_max"] = stamps
    elif args.kernel == "moe":
        from ..models import moe_all2all

        cfg, data, _, _ = contract.make_moe_inputs(args.experts, args.topk, args.hidden, args.tokens, 1, rank, ws, device="cuda",
                                                   dtype=getattr(torch, args.dtype), fixed_num_tokens=args.tokens,
                                                   routing=args.routing, weights="softmax")
        fn = lambda: moe_all2all.custom_kernel((cfg, data, rank, ws), mode=args.mode)  # noqa: E731
        times = timing.time_cuda(fn, warmup=3 if ws > 1 else 1, iters=args.iters, barrier=dist.barrier if ws > 1 else None)
        layer = moe_all2all.get_layer(cfg, rank, ws, mode=args.mode)
        if not args.few_launches:
            out["host_us"] = _host_time_us(fn, ws)
        if args.trace and layer.engine is not None:
            layer.enable_trace(True)
        y = fn()
        torch.cuda.synchronize()
        layer.check()
        ok, msg = oracle.check_moe_output(y, oracle.moe_expected_output(cfg, data, ws))
        out.update(config=[args.experts, args.topk, args.hidden, args.tokens], mode=layer.mode, us=[t * 1e3 for t in times],
                   ok=ok, msg=msg)
        if args.trace and layer.trace is not None:
            d, c = layer.trace[0].tolist(), layer.trace[1].tolist()
            names_d = ["start", "counted", "rows_issued", "counts_arrived", "metadata_stored", "all_sources_delivered",
                       "replicated", "last_cta_exit"]
            names_c = ["start", "weights_exchanged", "partials_pushed", "all_partials_arrived", "-", "-", "-", "last_cta_exit"]
            out["dispatch_trace_us"] = {nm: round((v - d[0]) / 1e3, 1) for nm, v in zip(names_d, d) if v > 0}
            out["combine_trace_us"] = {nm: round((v - d[0]) / 1e3, 1) for nm, v in zip(names_c, c) if v > 0 and nm != "-"}
    else:
        from ..ops.fp8_gemm import fp8_gemm, fp8_gemm_reference

        a = torch.randn(args.m, args.k, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn(args.n, args.k, device="cuda").to(torch.float8_e4m3fn)
        kb, nb = (args.k + 127) // 128, (args.n + 127) // 128
        a_s = torch.rand(args.m, kb, device="cuda") + 0.5
        b_s = torch.rand(nb, kb, device="cuda") + 0.5
        times = timing.time_cuda(lambda: fp8_gemm(a, b, a_s, b_s), warmup=1, iters=args.iters)
        c = fp8_gemm(a, b, a_s, b_s)
        out.update(shape=[args.m, args.n, args.k], us=[t * 1e3 for t in times],
                   tflops=2.0 * args.m * args.n * args.k / min(times) / 1e9,
                   rel_err=oracle.relative_error(c, fp8_gemm_reference(a, b, a_s, b_s)))
    torch.cuda.synchronize()
    print(json.dumps(out), flush=True)
    if ws > 1:
        _release()  # collective: nobody exits while a peer maps its slab or its memory is bound to a multicast object
        dist.barrier()
        dist.destroy_process_group()
    return 0


def _release() -> None:
    from .eval import release_workspaces

    release_workspaces()


if __name__ == "__main__":
    try:
        code = main()
    except Exception:
        try:
            _release()  # a rank that failed still takes its workspaces down together with the others
        except Exception:  # noqa: BLE001 - the original failure is the one to report
            pass
        raise
    sys.exit(code)
