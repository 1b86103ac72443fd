"""Peer-store bandwidth between the GPUs of one node, by mechanism.

Every rank pushes ``--mb`` megabytes from its own slab into a peer's slab with the probe
kernel of csrc/link_probe.cu and times it with CUDA events on the sender; the kernel ends
with a system-scope fence, so the time covers delivery.  Patterns:

* ``pair``   rank r -> rank r ^ 1, both directions at once (one busy link pair per GPU)
* ``oneway`` even ranks send to the next odd rank, odd ranks idle (one direction only)
* ``incast`` every rank but 0 sends to rank 0 (the hot-expert case of a skewed MoE dispatch)

The result is the denominator for the link-bound side of the rooflines.  The reference has
no counterpart (its transfers are library collectives, all2all/hipv8.py:281-359).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m amd_distributed_2025_b200.harness.link_probe --mb 256
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from ..parallel.symm_mem import SlabLayout, SymmetricWorkspace


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--mb", type=int, default=256)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--grids", default="148,296")
    args = ap.parse_args(argv)
    rank, ws = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if ws > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ..ops import _ext

    ext = _ext.load()
    nbytes = args.mb << 20
    lay = SlabLayout(ext.HEAP_HEADER_BYTES)
    lay.add("src", nbytes)
    lay.add("dst", nbytes * max(ws, 1))  # one landing area per sender
    ws_obj = SymmetricWorkspace(lay, rank=rank, world_size=ws)
    ws_obj.view("src", (nbytes,), torch.uint8).random_(0, 255)
    src_off, dst_off = lay.offset("src"), lay.offset("dst") + rank * nbytes
    patterns = {"pair": rank ^ 1 if (rank ^ 1) < ws else None,
                "oneway": rank + 1 if (rank % 2 == 0 and rank + 1 < ws) else None,
                "incast": 0 if rank != 0 else None}
    if ws == 1:
        patterns = {"local": 0}
    results = []
    for pattern, peer in patterns.items():
        for mode, chunk in ((0, 4096), (1, 2048), (1, 4096), (1, 8192)):
            for grid in [int(g) for g in args.grids.split(",")]:
                times = []
                for it in range(args.iters + 1):
                    torch.cuda.synchronize()
                    if ws > 1:
                        dist.barrier()
                    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record()
                    if peer is not None:
                        ws_obj.heap.link_probe(peer, src_off, dst_off, nbytes, mode, chunk, grid, ws_obj.wait_limit_ns)
                    stop.record()
                    torch.cuda.synchronize()
                    if it:
                        times.append(start.elapsed_time(stop))
                ws_obj.check(sync=True)
                if peer is not None:
                    results.append({"pattern": pattern, "rank": rank, "peer": peer, "mode": "lanes" if mode == 0 else f"bulk{chunk}",
                                    "grid": grid, "gb_per_s": round(nbytes / (min(times) * 1e-3) / 1e9, 1)})
    if ws > 1:
        gathered = [None] * ws
        dist.all_gather_object(gathered, results)
    else:
        gathered = [results]
    if rank == 0:
        table = {}
        for per_rank in gathered:
            for r in per_rank:
                table.setdefault((r["pattern"], r["mode"], r["grid"]), []).append(r["gb_per_s"])
        for (pattern, mode, grid), vals in sorted(table.items()):
            print(json.dumps({"pattern": pattern, "mode": mode, "grid": grid, "senders": len(vals), "min_gb_per_s": min(vals),
                              "max_gb_per_s": max(vals), "sum_gb_per_s": round(sum(vals), 1)}), flush=True)
    torch.cuda.synchronize()
    if ws > 1:
        dist.barrier()
    ws_obj.close(collective=True)
    if ws > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
