"""Row-parallel linear layer: GEMM (+bias) fused with reduce-scatter.

Contract of the reference (gemm-rs/reference.py:36-60, gemm-rs/submission.py:5-29):
``custom_kernel((input[M, K/ws], weight[N, K/ws], bias[N] | None)) -> out[M/ws, N]`` in
bf16, where ``out`` is this rank's row block of ``sum_r input_r @ weight_r.T`` plus the
bias.  The reference adds the bias on every rank *before* the reduction, so its checker
expects ``world_size * bias``; ``bias_mode="per_rank"`` (default) reproduces that,
``"once"`` adds the bias a single time.

``GemmRS`` owns the symmetric workspace of the fused kernel (csrc/gemm_rs_sm100.cu): two
parities of a bf16 staging buffer ``[world][M/ws][N]`` that peers store partial rows into
and two parities of per-tile arrival counters.  Calls alternate parity, which is what
lets consecutive calls overlap safely without any barrier between them.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..contract import GemmRsInput
from ..parallel.baseline_nccl import gemm_rs_torch
from ..parallel.symm_mem import SlabLayout, SymmetricWorkspace


def gemm_rs_slab_layout(max_m: int, max_n: int, world_size: int, header_bytes: int, ext) -> SlabLayout:
    stage_bytes, counter_bytes = ext.gemm_rs_workspace_bytes(max_m, max_n, world_size)
    lay = SlabLayout(header_bytes)
    lay.add("counters0", counter_bytes)
    lay.add("counters1", counter_bytes)
    lay.add("stage0", stage_bytes)
    lay.add("stage1", stage_bytes)
    return lay


class GemmRS:
    def __init__(
        self,
        max_m: int,
        max_n: int,
        rank: Optional[int] = None,
        world_size: Optional[int] = None,
        group=None,
        device: Optional[torch.device] = None,
        wait_limit_ms: Optional[float] = None,
    ):
        from ..ops import _ext

        self.ext = _ext.load()
        initialized = dist.is_available() and dist.is_initialized()
        self.world_size = world_size if world_size is not None else (dist.get_world_size(group) if initialized else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if initialized else 0)
        self.max_m, self.max_n = int(max_m), int(max_n)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        layout = gemm_rs_slab_layout(self.max_m, self.max_n, self.world_size, self.ext.HEAP_HEADER_BYTES, self.ext)
        self.ws = SymmetricWorkspace(
            layout,
            rank=self.rank,
            world_size=self.world_size,
            group=group,
            device=self.device,
            wait_limit_ms=wait_limit_ms,
        )
        self.max_ctas = 0  # 0 = one CTA per SM
        self.block_n = 0  # 0 = tile width chosen from the shape (64 / 128 / 256)
        self.cta_pair = -1  # -1 = chosen from the shape; 0 = single CTAs; 1 = CTA pairs (256-row tiles)

    def __call__(
        self,
        a: torch.Tensor,
        w: torch.Tensor,
        bias: Optional[torch.Tensor] = None,
        bias_mode: str = "per_rank",
        out: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        m, n = a.shape[0], w.shape[0]
        stage_bytes, counter_bytes = self.ext.gemm_rs_workspace_bytes(m, n, self.world_size)
        if stage_bytes > self.ws.layout.size("stage0") or counter_bytes > self.ws.layout.size("counters0"):
            raise ValueError(f"problem {m}x{n} exceeds the workspace capacity {self.max_m}x{self.max_n}")
        if bias_mode not in ("per_rank", "once"):
            raise ValueError("bias_mode must be 'per_rank' or 'once'")
        self.ws.check()
        if out is None:
            out = torch.empty((m // self.world_size, n), dtype=torch.bfloat16, device=a.device)
        epoch = self.ws.next_epoch("gemm_rs")
        parity = epoch & 1
        # "per_rank": every rank adds the bias to its rounded partial before the reduction
        # (the reference's order of operations); "once": the owner adds it after the sum.
        at_source = bias_mode == "per_rank"
        self.ext.gemm_rs(
            self.ws.heap,
            a.contiguous(),
            w.contiguous(),
            bias,
            out,
            1.0,
            at_source,
            self.ws.offset(f"stage{parity}"),
            self.ws.offset(f"counters{parity}"),
            epoch,
            self.ws.wait_limit_ns,
            self.max_ctas,
            self.block_n,
            self.cta_pair,
        )
        return out

    def check(self, sync: bool = True) -> None:
        self.ws.check(sync)

    def close(self) -> None:
        self.ws.close()


_OPS: Dict[tuple, GemmRS] = {}


def get_op(m: int, n: int, group=None) -> GemmRS:
    """Cached operator whose workspace fits ``[m, n]``; growing it is collective."""
    initialized = dist.is_available() and dist.is_initialized()
    ws = dist.get_world_size(group) if initialized else 1
    key = (ws, id(group), torch.cuda.current_device())
    op = _OPS.get(key)
    if op is not None:
        stage_bytes, counter_bytes = op.ext.gemm_rs_workspace_bytes(m, n, ws)
        if stage_bytes <= op.ws.layout.size("stage0") and counter_bytes <= op.ws.layout.size("counters0"):
            return op
        torch.cuda.synchronize()
        if initialized:
            dist.barrier(group=group)
        op.close()
        m, n = max(m, op.max_m), max(n, op.max_n)
    op = GemmRS(m, n, group=group)
    _OPS[key] = op
    return op


def release_ops() -> None:
    for op in _OPS.values():
        op.close()
    _OPS.clear()


def custom_kernel(data: GemmRsInput, bias_mode: str = "per_rank", backend: str = "auto") -> torch.Tensor:
    """``[M/ws, N]`` bf16 result of the row-parallel linear layer (gemm-rs/reference.py:36-60)."""
    a, w, bias = data
    if backend == "torch" or (backend == "auto" and not a.is_cuda):
        if bias_mode == "once" and bias is not None and dist.is_initialized():
            out = gemm_rs_torch((a, w, None))
            return out + bias
        return gemm_rs_torch(data)
    with torch.cuda.device(a.device):
        op = get_op(a.shape[0], w.shape[0])
        return op(a, w, bias, bias_mode)
