"""Device-side timing helpers.

Rules followed everywhere a number is reported: warm-up iterations first, CUDA events on
the launching stream, a synchronize on both sides of the timed region, the L2 flushed
between iterations (a write larger than the 126 MB L2), and for multi-rank runs the
maximum over ranks.  The reference leaves timing to an evaluator that is not part of its
tree (all2all/task.yml:6-8).
"""
from __future__ import annotations

import math
import statistics
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

L2_FLUSH_BYTES = 256 * 1024 * 1024
_flush_buf: Dict[int, torch.Tensor] = {}


def flush_l2(device: Optional[torch.device] = None) -> None:
    """Overwrite a buffer larger than L2 so the next kernel starts from a cold cache."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    buf = _flush_buf.get(dev)
    if buf is None:
        buf = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=f"cuda:{dev}")
        _flush_buf[dev] = buf
    buf.zero_()


def time_cuda(
    fn: Callable[[], object],
    warmup: int = 3,
    iters: int = 10,
    flush: bool = True,
    barrier: Optional[Callable[[], None]] = None,
) -> List[float]:
    """Per-iteration device time of ``fn`` in milliseconds.

    ``barrier`` (e.g. ``dist.barrier``) is called before every timed iteration so that all
    ranks enter together; it is outside the timed events.
    """
    for _ in range(max(warmup, 0)):
        fn()
    torch.cuda.synchronize()
    times: List[float] = []
    for _ in range(iters):
        if flush:
            flush_l2()
        if barrier is not None:
            barrier()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    return times


def max_over_ranks(values: List[float], group=None) -> List[float]:
    """Element-wise maximum of a list of per-iteration times over all ranks."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return list(values)
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.tolist()


def summarize(times_ms: List[float]) -> Dict[str, float]:
    s = sorted(times_ms)
    return {
        "mean_ms": statistics.fmean(s),
        "median_ms": statistics.median(s),
        "min_ms": s[0],
        "max_ms": s[-1],
        "n": len(s),
    }


def geomean(values: List[float]) -> float:
    """Geometric mean, the ranking rule of both tasks (all2all/task.yml:68, gemm-rs/task.yml:62)."""
    vals = [v for v in values if v > 0]
    if not vals:
        return float("nan")
    return math.exp(sum(math.log(v) for v in vals) / len(vals))
