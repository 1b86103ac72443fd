"""The two operators for CPU ranks of one node, without a collective library.

``HostMoEAllToAll`` and ``HostGemmRS`` have the interfaces of ``MoEAllToAll`` and
``GemmRS`` and run the same one-sided protocols, in C++ over shared memory
(csrc/host_ops.cpp): dispatch publishes per-expert counts, derives every row's slot and
writes the row into the owner's ``expert_x``; combine pulls rows out of the owners'
``expert_y`` ("direct"); with ``mode="dedup"`` a token's row lands once per destination rank
with a record of its final rows, the owner copies it into ``expert_x`` itself, and combine
returns one pre-reduced row per (token, owner) -- the device kernels' default protocol
(csrc/moe_dedup.cu); GEMM + reduce-scatter stores partial row blocks into the owners' staging
slots, alternating between two parities so that calls need no barrier between them.

The reference's CPU path is its oracle (all2all/reference.py:63-272,
gemm-rs/reference.py:52-59): per-row Python around gloo collectives.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..contract import META_DIM, GemmRsInput, MoEConfig, MoEInput
from ..parallel.host_symm import HostSymmetricWorkspace, shared_prefix
from .gemm_rs import gemm_rs_slab_layout
from .moe_all2all import MODES, moe_slab_layout


def default_host_mode() -> str:
    """Protocol of the CPU MoE layer: ``B200_HOST_MOE_MODE`` or "direct".  Between processes of one
    node every copy is a memory copy, so sending a token once per destination rank saves nothing
    there; "dedup" exists on CPU ranks to run the device kernels' default protocol (records, chunk
    flags, owner-side pre-reduction) under real concurrency."""
    mode = os.environ.get("B200_HOST_MOE_MODE", "direct").strip().lower()
    if mode not in MODES:
        raise ValueError(f"B200_HOST_MOE_MODE={mode!r}: expected one of {MODES}")
    return mode


def _check_peers(monitor) -> None:
    """With a monitor: post a heartbeat and raise ``PeerLostError`` if a peer announced its
    departure or fell silent -- before this rank starts waiting for it."""
    if monitor is not None:
        monitor.beat()
        monitor.assert_all_alive()


class HostMoEAllToAll:
    """MoE dispatch / expert op / combine between CPU ranks through shared memory."""

    META_DIM = META_DIM

    def __init__(self, cfg: MoEConfig, rank: int, world_size: int, prefix: Optional[str] = None, group=None,
                 wait_limit_ms: Optional[float] = None, monitor=None, mode: Optional[str] = None, chunks: int = 1,
                 partial_dtype: Optional[torch.dtype] = None):
        from ..ops import _ext

        self.ext = _ext.load()
        self.monitor = monitor  # optional parallel.health.HealthMonitor, consulted before every step that waits on peers
        if cfg.num_experts % world_size:
            raise ValueError("num_experts must divide by the world size")
        self.mode = default_host_mode() if mode is None else mode
        if self.mode not in MODES:
            raise ValueError(f"mode {self.mode!r}: expected one of {MODES}")
        if self.mode == "dedup" and cfg.experts_per_token > 15:
            raise ValueError("the dedup protocol keeps a token's entries in one 32-word record: at most 15 experts per token")
        if partial_dtype not in (None, cfg.out_dtype, torch.float32):
            raise ValueError("partial_dtype must be the output type or float32")
        self.partial_fp32 = partial_dtype == torch.float32 and cfg.out_dtype != torch.float32
        self.chunks = max(1, min(8, int(chunks)))  # dedup: flags per dispatch, so owners replicate while rows still arrive
        self.cfg, self.rank, self.world_size = cfg, rank, world_size
        self.num_local_experts = cfg.num_local_experts(world_size)
        self.max_recv = cfg.max_recv(world_size)
        layout = moe_slab_layout(cfg, world_size, self.ext.HEAP_HEADER_BYTES, mode=self.mode,
                                 partial_bytes=4 if self.partial_fp32 else 0)
        self.ws = HostSymmetricWorkspace(layout, prefix or shared_prefix(group, "moe"), rank, world_size, wait_limit_ms)
        self._offsets = [layout.offset(n) for n in ("counts", "expert_x", "expert_meta", "expert_y")]
        self._dedup_offsets = ([layout.offset(n) for n in ("counts", "expert_x", "expert_meta", "expert_y", "land", "tok_rec", "ret")]
                               if self.mode == "dedup" else None)
        self._dispatch_epoch = 0
        cells = (self.num_local_experts, self.max_recv)
        self.expert_x = self.ws.view("expert_x", (*cells, cfg.hidden_dim), cfg.in_dtype)
        self.expert_meta = self.ws.view("expert_meta", (*cells, META_DIM), torch.int32)
        self.expert_y = self.ws.view("expert_y", (*cells, cfg.hidden_dim), cfg.out_dtype)
        # int32 [tokens * k, 3]: owner, local expert, slot ("direct"); [tokens * k, 2]: owner, row on the owner ("dedup")
        self.route: Optional[torch.Tensor] = None
        self.expert_num_tokens: Optional[torch.Tensor] = None

    def dispatch(self, dp_x: torch.Tensor, indices: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """``(expert_num_tokens, expert_x, expert_meta)`` as all2all/reference.py:63-164 returns
        them; the two buffers are views of this rank's slab."""
        cfg = self.cfg
        if dp_x.dtype != cfg.in_dtype or dp_x.shape[1] != cfg.hidden_dim:
            raise ValueError("dp_x does not match the configuration")
        if indices.shape[0] > cfg.max_num_tokens:
            raise ValueError(f"{indices.shape[0]} tokens exceed max_num_tokens={cfg.max_num_tokens}")
        _check_peers(self.monitor)
        # No guard is needed for a dispatch that follows a dispatch: in both protocols a rank stores
        # nothing on a peer before it has every rank's counts of the new call, and a rank publishes
        # those only when its caller has entered the new call, i.e. is done with the old buffers.
        if self.mode == "dedup":
            self._dispatch_epoch = self.ws.next_epoch("moe_dispatch")
            status, route, num = self.ext.host_moe_dedup_dispatch(
                self.ws.heap, self._dedup_offsets, dp_x.contiguous(), indices, cfg.num_experts, self.max_recv,
                cfg.max_num_tokens, cfg.out_dtype, self.chunks, self._dispatch_epoch, self.ws.wait_limit_ns,
            )
        else:
            status, route, num = self.ext.host_moe_dispatch(
                self.ws.heap, self._offsets, dp_x.contiguous(), indices, cfg.num_experts, self.max_recv, cfg.out_dtype,
                self.ws.next_epoch("moe_dispatch"), self.ws.wait_limit_ns,
            )
        self.ws.raise_on(status)
        self.route, self.expert_num_tokens = route, num
        return num, self.expert_x, self.expert_meta

    def expert_scale(self, scale: float, expert_num_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The task's stand-in expert (all2all/reference.py:265): ``expert_y = expert_x * scale``
        over the rows that hold tokens; returns the ``expert_y`` view."""
        cfg = self.cfg
        num = self.expert_num_tokens if expert_num_tokens is None else expert_num_tokens
        self.ext.host_moe_expert_scale(
            self.ws.heap, self._offsets, cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim, self.max_recv,
            cfg.in_dtype, cfg.out_dtype, num.to(torch.int32).contiguous(), float(scale),
        )
        return self.expert_y

    def combine(self, out_tokens: torch.Tensor, weights: torch.Tensor, expert_y: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Weighted sum over k of every token's expert outputs into ``out_tokens[:tokens]``.
        ``expert_y`` other than the workspace's own buffer is copied into it first."""
        if self.route is None:
            raise RuntimeError("combine needs the route table of a preceding dispatch")
        cfg = self.cfg
        if self.mode == "dedup":
            # the owner reduces its own expert outputs: any local tensor of the dispatch layout will do
            y = self.expert_y if expert_y is None else expert_y
            if y.shape != self.expert_y.shape or y.dtype != cfg.out_dtype:
                raise ValueError("expert_y does not have the dispatch layout / out_dtype")
            _check_peers(self.monitor)
            status = self.ext.host_moe_dedup_combine(
                self.ws.heap, self._dedup_offsets, cfg.num_experts, self.max_recv, cfg.max_num_tokens, cfg.in_dtype,
                self.partial_fp32, self.route, weights.to(torch.float32).contiguous(), y.contiguous(), out_tokens,
                self._dispatch_epoch, self.ws.next_epoch("moe_combine"), self.ws.wait_limit_ns,
            )
            self.ws.raise_on(status)
            return out_tokens
        if expert_y is not None and expert_y.data_ptr() != self.expert_y.data_ptr():
            self.expert_y.copy_(expert_y)
        _check_peers(self.monitor)
        status = self.ext.host_moe_combine(
            self.ws.heap, self._offsets, cfg.num_experts, self.max_recv, cfg.in_dtype, self.route,
            weights.to(torch.float32).contiguous(), out_tokens, self.ws.next_epoch("moe_combine"), self.ws.wait_limit_ns,
        )
        self.ws.raise_on(status)
        return out_tokens

    def forward(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, scale: float) -> torch.Tensor:
        self.dispatch(x, indices)
        self.expert_scale(scale)
        y = torch.empty((indices.shape[0], self.cfg.hidden_dim), dtype=self.cfg.out_dtype)
        return self.combine(y, weights)

    def close(self) -> None:
        self.ws.close()


class HostGemmRS:
    """GEMM (+bias) + reduce-scatter between CPU ranks: library matmul per rank, then the
    partial row blocks go straight into the owners' staging slots."""

    def __init__(self, stage_bytes: int, rank: int, world_size: int, prefix: Optional[str] = None, group=None,
                 wait_limit_ms: Optional[float] = None, monitor=None):
        from ..ops import _ext

        self.ext = _ext.load()
        self.monitor = monitor
        self.rank, self.world_size, self.stage_bytes = rank, world_size, int(stage_bytes)
        layout = gemm_rs_slab_layout(self.stage_bytes, 0, self.ext.HEAP_HEADER_BYTES)
        self.ws = HostSymmetricWorkspace(layout, prefix or shared_prefix(group, "rs"), rank, world_size, wait_limit_ms)

    def __call__(self, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 bias_mode: str = "per_rank") -> torch.Tensor:
        if bias_mode not in ("per_rank", "once"):
            raise ValueError("bias_mode must be 'per_rank' or 'once'")
        _check_peers(self.monitor)
        partial = torch.matmul(a, w.T)
        if bias is not None and bias_mode == "per_rank":
            partial = partial + bias  # the reference's order: every rank adds it before the reduction
        epoch = self.ws.next_epoch("gemm_rs")
        status, out = self.ext.host_reduce_scatter(
            self.ws.heap, self.ws.offset(f"stage{epoch & 1}"), self.stage_bytes, partial.contiguous(),
            bias if bias_mode == "once" else None, epoch, self.ws.wait_limit_ns,
        )
        self.ws.raise_on(status)
        return out

    def close(self) -> None:
        self.ws.close()


# --------------------------------------------------------------------------------------
# cached operators behind the task entry points
# --------------------------------------------------------------------------------------

_LAYERS: Dict[tuple, HostMoEAllToAll] = {}
_OPS: Dict[tuple, HostGemmRS] = {}


def get_layer(cfg: MoEConfig, rank: int, world_size: int, group=None, mode: Optional[str] = None) -> HostMoEAllToAll:
    """Cached layer for ``cfg``; creating one is collective (the ranks agree on a name)."""
    mode = default_host_mode() if mode is None else mode
    key = (cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim, cfg.max_num_tokens, cfg.in_dtype, cfg.out_dtype,
           rank, world_size, id(group), mode)
    layer = _LAYERS.get(key)
    if layer is None:
        layer = _LAYERS[key] = HostMoEAllToAll(cfg, rank, world_size, group=group, mode=mode)
    return layer


def get_op(m: int, n: int, elem_bytes: int, group=None) -> HostGemmRS:
    initialized = dist.is_available() and dist.is_initialized()
    ws = dist.get_world_size(group) if initialized else 1
    rank = dist.get_rank(group) if initialized else 0
    key = (ws, id(group))
    need = m * n * elem_bytes
    op = _OPS.get(key)
    if op is None or op.stage_bytes < need:
        if op is not None:
            if initialized:
                dist.barrier(group=group)  # nobody may still be reading the old slabs
            op.close()
        op = _OPS[key] = HostGemmRS(need, rank, ws, group=group)
    return op


def release() -> None:
    """Unmap and unlink every cached slab (all ranks, while idle)."""
    for cache in (_LAYERS, _OPS):
        for op in cache.values():
            op.close()
        cache.clear()


def moe_custom_kernel(data: MoEInput, mode: Optional[str] = None) -> torch.Tensor:
    """``custom_kernel`` of the MoE task on CPU ranks (all2all/reference.py:256-272)."""
    cfg, rank_data, rank, world_size = data
    layer = get_layer(cfg, rank, world_size, mode=mode)
    n = rank_data.num_tokens
    return layer.forward(rank_data.x, rank_data.indices[:n], rank_data.weights[:n], 1 + rank)


def gemm_rs_custom_kernel(data: GemmRsInput, bias_mode: str = "per_rank") -> torch.Tensor:
    """``custom_kernel`` of the GEMM + reduce-scatter task on CPU ranks (gemm-rs/reference.py:36-60)."""
    a, w, bias = data
    op = get_op(a.shape[0], w.shape[0], a.element_size())
    return op(a, w, bias, bias_mode)
