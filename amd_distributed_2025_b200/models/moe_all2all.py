"""MoE expert-parallel layer: dispatch -> expert op -> combine over NVLink peer memory.

Same contract as the reference solution (all2all/hipv8.py:254-394, oracle
all2all/reference.py:55-272):

* ``MoEAllToAll(cfg, rank, world_size)`` with
  ``dispatch(dp_x, indices) -> (expert_num_tokens, expert_x, expert_meta)`` and
  ``combine(out_tokens, weights, expert_meta, expert_y, expert_num_tokens, num_tokens)``;
* ``custom_kernel((cfg, rank_data, rank, world_size)) -> y[num_tokens, hidden]``.

Differences in mechanism, not in results: the three returned tensors are views of this
rank's symmetric workspace, in the reference's row order (source rank, token, k), and
nothing in a call synchronises with the host.  Two protocols fill them (``mode``, default
from ``B200_MOE_MODE``):

* ``"dedup"`` (default, csrc/moe_dedup.cu): a token crosses NVLink once per destination
  *rank*; the owner replicates the landed row into ``expert_x[e_local, slot]`` locally.
  Combine runs on the owner: per (source, token) it forms the weighted sum over its local
  experts in fp32 and pushes that one row back; the source adds the rows of the owners it
  used.  ``partial_dtype=torch.float32`` makes those rows travel un-rounded.
* ``"direct"`` (csrc/moe_kernels.cu): one row per (token, k) entry, stored by the sender
  straight into the owner's ``expert_x``; combine pulls ``expert_y`` rows from the owners
  with the route table that dispatch recorded.

Calls alternate ``dispatch`` and ``combine`` (or use ``forward``); every rank issues the
same sequence.

On CPU tensors (or ``backend="torch"``) the layer falls back to the library-collective
implementation in ``parallel/baseline_nccl.py``; that is how the fp32 two-rank CPU
configuration runs.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..contract import META_DIM, MoEConfig, MoEInput
from ..parallel.baseline_nccl import TorchAllToAll
from ..parallel.symm_mem import SlabLayout, SymmetricWorkspace, checked_guard_bytes

_DTYPE_SIZE = {torch.float16: 2, torch.bfloat16: 2, torch.float32: 4}


MODES = ("dedup", "direct")


def default_mode() -> str:
    mode = os.environ.get("B200_MOE_MODE", "dedup").strip().lower()
    if mode not in MODES:
        raise ValueError(f"B200_MOE_MODE={mode!r}: expected one of {MODES}")
    return mode


def moe_slab_layout(cfg: MoEConfig, world_size: int, header_bytes: int, mode: str = "direct",
                    partial_bytes: int = 0, guard_bytes: int = 0) -> SlabLayout:
    """Offsets of the MoE regions inside every rank's slab.  The "dedup" protocol adds the
    landing buffer, the per-(source, token) row lists / weights / marks and the return buffer."""
    e_local = cfg.num_local_experts(world_size)
    max_recv = cfg.max_recv(world_size)
    rows = e_local * max_recv
    lay = SlabLayout(header_bytes, guard_bytes=guard_bytes)
    lay.add("counts", world_size * cfg.num_experts * 4)
    lay.add("expert_meta", rows * META_DIM * 4)
    lay.add("expert_x", rows * cfg.hidden_dim * _DTYPE_SIZE[cfg.in_dtype])
    lay.add("expert_y", rows * cfg.hidden_dim * _DTYPE_SIZE[cfg.out_dtype])
    if mode == "dedup":
        toks = world_size * cfg.max_num_tokens
        lay.add("land", toks * cfg.hidden_dim * _DTYPE_SIZE[cfg.in_dtype])
        rec_ints = (1 + 2 * cfg.experts_per_token + 3) // 4 * 4  # mark, k rows, k weights, padded to 16 bytes
        lay.add("tok_rec", toks * rec_ints * 4)
        lay.add("ret", toks * cfg.hidden_dim * (partial_bytes or _DTYPE_SIZE[cfg.out_dtype]))
    return lay


class MoEAllToAll:
    META_DIM = META_DIM

    def __init__(
        self,
        cfg: MoEConfig,
        rank: int,
        world_size: int,
        group=None,
        device: Optional[torch.device] = None,
        wait_limit_ms: Optional[float] = None,
        mode: Optional[str] = None,
        partial_dtype: Optional[torch.dtype] = None,
        monitor=None,
    ):
        if cfg.in_dtype not in _DTYPE_SIZE or cfg.out_dtype not in _DTYPE_SIZE:
            raise ValueError("in_dtype / out_dtype must be float16, bfloat16 or float32")
        if cfg.in_dtype != cfg.out_dtype:
            # the reference converts with expert_x.to(out_dtype) (all2all/reference.py:262); its generator
            # only ever produces equal types, and the device kernels move rows as bytes
            raise ValueError(f"in_dtype {cfg.in_dtype} != out_dtype {cfg.out_dtype}: the GPU layer needs equal types")
        self.mode = mode or default_mode()
        if self.mode not in MODES:
            raise ValueError(f"mode {self.mode!r}: expected one of {MODES}")
        if partial_dtype not in (None, cfg.out_dtype, torch.float32):
            raise ValueError("partial_dtype must be the output type or float32")
        self.partial_fp32 = partial_dtype == torch.float32 and cfg.out_dtype != torch.float32
        if cfg.experts_per_token > 15 and self.mode == "dedup":
            raise ValueError("the dedup protocol handles at most 15 experts per token (use mode='direct')")
        self.monitor = monitor  # optional parallel.health.HealthMonitor: peers are checked before every launch
        self.cfg = cfg
        self.rank = rank
        self.world_size = world_size
        self.group = group
        self.num_local_experts = cfg.num_local_experts(world_size)
        self.max_recv = cfg.max_recv(world_size)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())

        from ..ops import _ext

        ext = _ext.load()
        self.ext = ext
        layout = moe_slab_layout(cfg, world_size, ext.HEAP_HEADER_BYTES, self.mode,
                                 4 if self.partial_fp32 else 0, guard_bytes=checked_guard_bytes())
        self.ws = SymmetricWorkspace(
            layout, rank=rank, world_size=world_size, group=group, device=self.device, wait_limit_ms=wait_limit_ms
        )
        shape3 = (self.num_local_experts, self.max_recv, cfg.hidden_dim)
        self.expert_x = self.ws.view("expert_x", shape3, cfg.in_dtype)
        self.expert_y = self.ws.view("expert_y", shape3, cfg.out_dtype)
        self.expert_meta = self.ws.view("expert_meta", (self.num_local_experts, self.max_recv, META_DIM), torch.int32)
        n_max = max(cfg.max_num_tokens * cfg.experts_per_token, 1)
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        i32 = dict(dtype=torch.int32, device=self.device)
        self._blk_hist = torch.zeros(2 * sms * cfg.num_experts, **i32)
        self._local_rank = torch.zeros(n_max, **i32)
        self._route = torch.full((n_max, 2), -1, **i32)
        self.expert_num_tokens = torch.zeros(self.num_local_experts, **i32)
        self._num_tokens = 0
        self._dispatch_pending = False  # a dispatch whose combine has not run yet
        self._off_counts = self.ws.offset("counts")
        self._off_expert_x = self.ws.offset("expert_x")
        self._off_expert_meta = self.ws.offset("expert_meta")
        self._off_expert_y = self.ws.offset("expert_y")
        self.engine = None
        if self.mode == "dedup":
            names = ("counts", "expert_x", "expert_meta", "expert_y", "land", "tok_rec", "ret")
            self.engine = ext.MoeDedupEngine(
                self.ws.heap, cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim, cfg.max_num_tokens, self.max_recv,
                cfg.in_dtype, self.partial_fp32, [self.ws.offset(nm) for nm in names], self.expert_y, self._blk_hist,
                self._route, self.expert_num_tokens, self.ws.wait_limit_ns,
            )
            # B200_MOE_LANDING=lanes: rows cross NVLink as 16-byte stores from registers instead of bulk copies
            self.engine.bulk_landing = os.environ.get("B200_MOE_LANDING", "bulk").strip().lower() != "lanes"
            # B200_MOE_CHUNKS: chunks (1..8) a large dispatch is cut into so that replication overlaps the transfer
            self.engine.chunks = max(1, min(8, int(os.environ.get("B200_MOE_CHUNKS", "4"))))
            self.engine.chunk_min_ranks = int(os.environ.get("B200_MOE_CHUNK_MIN_RANKS", "4"))
            self.engine.chunk_min_bytes = int(os.environ.get("B200_MOE_CHUNK_MIN_BYTES", str(8 << 20)))
        self.trace: Optional[Tuple[torch.Tensor, torch.Tensor]] = None

    def _guard(self) -> None:
        """Host-side checks before a launch that waits on peers: an earlier device failure, and
        (with a monitor) peers that announced their departure or stopped their heartbeat."""
        self.ws.check()
        if self.monitor is not None:
            self.monitor.beat()
            self.monitor.assert_all_alive()

    def _quiesce_before_second_dispatch(self) -> None:
        """The dedup buffers are reused without a barrier because calls alternate dispatch and
        combine: a rank enters the next dispatch only after a combine in which every rank took
        part, i.e. after every owner has read what the next dispatch overwrites.  A dispatch that
        follows a dispatch has no such rendezvous behind it: the small kernel sends its rows before
        it has the peers' counts, so a fast sender could land new rows while a slow owner still
        replicates the previous ones.  This unusual sequence pays a device synchronisation and a
        host barrier instead.  (The "direct" kernels and the large dedup kernel store nothing on a
        peer before they have every rank's counts of the new call, which a rank publishes only
        once it has entered that call: they need no guard.)"""
        if self._dispatch_pending and self.world_size > 1 and self.engine is not None:
            torch.cuda.synchronize(self.device)
            if dist.is_available() and dist.is_initialized():
                dist.barrier(group=self.group)

    def enable_trace(self, on: bool = True) -> None:
        """Record ``globaltimer`` phase stamps (ns) of the next dedup calls: ``trace[0]`` dispatch =
        start, counted, rows issued, counts arrived, metadata stored, all sources delivered,
        replicated, last CTA exit; ``trace[1]`` combine = start, weights exchanged, partials
        pushed, all partials arrived, -, -, -, last CTA exit."""
        if self.engine is None:
            raise RuntimeError("phase stamps exist in the dedup kernels only")
        if on:
            self.trace = (torch.zeros(8, dtype=torch.int64, device=self.device),
                          torch.zeros(8, dtype=torch.int64, device=self.device))
            self.engine.set_trace(self.trace[0], self.trace[1])
        else:
            self.trace = None
            self.engine.set_trace(None, None)

    # -- dispatch ----------------------------------------------------------------------
    def dispatch(self, dp_x: torch.Tensor, indices: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        cfg = self.cfg
        if dp_x.shape[0] > cfg.max_num_tokens:
            raise ValueError(f"{dp_x.shape[0]} tokens exceed max_num_tokens={cfg.max_num_tokens}")
        if dp_x.shape[1] != cfg.hidden_dim or indices.shape[1] != cfg.experts_per_token:
            raise ValueError("dp_x / indices do not match the configuration")
        if dp_x.dtype != cfg.in_dtype:
            raise ValueError(f"dp_x is {dp_x.dtype}, configuration says {cfg.in_dtype}")
        self._guard()
        x = dp_x.contiguous()
        idx = indices.to(torch.int32).contiguous()
        self._num_tokens = x.shape[0]
        self._quiesce_before_second_dispatch()
        self._dispatch_pending = True
        if self.engine is not None:
            if self.engine.dispatch(x, idx):
                self.ws.check()
            return self.expert_num_tokens, self.expert_x, self.expert_meta
        self.ext.moe_dispatch(
            self.ws.heap,
            x,
            idx,
            cfg.num_experts,
            self.max_recv,
            self.ws.offset("counts"),
            self.ws.offset("expert_x"),
            self.ws.offset("expert_meta"),
            self._blk_hist,
            self._local_rank,
            self._route,
            self.expert_num_tokens,
            self.ws.next_epoch("moe_dispatch"),
            self.ws.wait_limit_ns,
        )
        return self.expert_num_tokens, self.expert_x, self.expert_meta

    # -- expert op of the task ---------------------------------------------------------
    def expert_scale(self, scale: float) -> torch.Tensor:
        """``expert_y = expert_x * scale`` on the rows dispatch delivered
        (all2all/reference.py:262 with ``scale = 1 + rank``)."""
        self.ext.moe_expert_scale(self.expert_x, self.expert_y, self.expert_num_tokens, float(scale))
        return self.expert_y

    # -- combine -----------------------------------------------------------------------
    def combine(
        self,
        out_tokens: torch.Tensor,
        weights: torch.Tensor,
        expert_meta: torch.Tensor,
        expert_y: torch.Tensor,
        expert_num_tokens: torch.Tensor,
        num_tokens: Optional[int] = None,
        accumulate: bool = False,
    ) -> torch.Tensor:
        """Weighted top-k sum of the expert outputs back into token order.

        ``expert_meta`` / ``expert_num_tokens`` are accepted for interface parity; routing
        comes from the table recorded by the preceding ``dispatch``.  ``expert_y`` may be
        any tensor of the dispatch layout: if it is not this layer's symmetric buffer its
        valid rows are first copied there so that peers can read them.  Rows
        ``[0, num_tokens)`` of ``out_tokens`` are overwritten (``accumulate=True`` adds
        instead, which equals the reference's ``+=`` onto a caller-provided buffer).
        """
        n = self._num_tokens if num_tokens is None else int(num_tokens)
        if n != self._num_tokens:
            raise ValueError("num_tokens differs from the preceding dispatch")
        self._guard()
        self._dispatch_pending = False
        if self.engine is not None:
            # the owner reduces its own expert outputs, so any local tensor of the dispatch layout will do
            if expert_y.shape != self.expert_y.shape or expert_y.dtype != self.expert_y.dtype:
                raise ValueError("expert_y does not have the dispatch layout / out_dtype")
            target = out_tokens
            if accumulate or not out_tokens.is_contiguous() or out_tokens.dtype != self.cfg.out_dtype:
                target = torch.empty((max(n, 1), self.cfg.hidden_dim), dtype=self.cfg.out_dtype, device=out_tokens.device)
            if self.engine.combine(target, weights.to(torch.float32).contiguous(), expert_y.contiguous()):
                self.ws.check()
            if target is not out_tokens:
                if accumulate:
                    out_tokens[:n] += target[:n].to(out_tokens.dtype)
                else:
                    out_tokens[:n] = target[:n].to(out_tokens.dtype)
            return out_tokens
        if expert_y.data_ptr() != self.expert_y.data_ptr():
            if expert_y.shape != self.expert_y.shape or expert_y.dtype != self.expert_y.dtype:
                raise ValueError("expert_y does not have the dispatch layout / out_dtype")
            self.ext.moe_expert_scale(expert_y.contiguous(), self.expert_y, self.expert_num_tokens, 1.0)
        target = out_tokens
        if accumulate or not out_tokens.is_contiguous() or out_tokens.dtype != self.cfg.out_dtype:
            target = torch.empty((max(n, 1), self.cfg.hidden_dim), dtype=self.cfg.out_dtype, device=out_tokens.device)
        self.ext.moe_combine(
            self.ws.heap,
            target,
            weights.to(torch.float32).contiguous(),
            self._route,
            n,
            self.max_recv,
            self.ws.offset("expert_y"),
            self.ws.next_epoch("moe_combine"),
            self.ws.wait_limit_ns,
        )
        if target is not out_tokens:
            if accumulate:
                out_tokens[:n] += target[:n].to(out_tokens.dtype)
            else:
                out_tokens[:n] = target[:n].to(out_tokens.dtype)
        return out_tokens

    # -- the task pipeline in one native call -------------------------------------------
    def forward(self, dp_x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, scale: float) -> torch.Tensor:
        """dispatch -> ``expert_y = expert_x * scale`` -> combine, launched back to back from
        one native call.  In "dedup" mode the scale is applied while the landed rows are
        replicated into the expert buffers (two launches); in "direct" mode it is the three
        kernels of the separate methods."""
        cfg = self.cfg
        if dp_x.shape[0] > cfg.max_num_tokens or dp_x.shape[1] != cfg.hidden_dim or dp_x.dtype != cfg.in_dtype:
            raise ValueError("dp_x does not match the configuration")
        if indices.shape[1] != cfg.experts_per_token:
            raise ValueError("indices do not match the configuration")
        if self.monitor is not None:
            self.monitor.beat()
            self.monitor.assert_all_alive()
        x = dp_x if dp_x.is_contiguous() else dp_x.contiguous()
        idx = indices if (indices.dtype == torch.int32 and indices.is_contiguous()) else indices.to(torch.int32).contiguous()
        w = weights if (weights.dtype == torch.float32 and weights.is_contiguous()) else weights.to(torch.float32).contiguous()
        self._num_tokens = x.shape[0]
        out = torch.empty((x.shape[0], cfg.hidden_dim), dtype=cfg.out_dtype, device=x.device)
        self._quiesce_before_second_dispatch()
        self._dispatch_pending = False
        if self.engine is not None:
            if self.engine.forward(x, idx, w, out, float(scale)):
                self.ws.check()  # an earlier kernel recorded a failure: raise it
            return out
        self.ws.check()
        self.ext.moe_forward(
            self.ws.heap, x, idx, w, out, cfg.num_experts, self.max_recv,
            self._off_counts, self._off_expert_x, self._off_expert_meta, self._off_expert_y,
            self.expert_x, self.expert_y, self._blk_hist, self._local_rank, self._route, self.expert_num_tokens,
            float(scale), self.ws.next_epoch("moe_dispatch"), self.ws.next_epoch("moe_combine"), self.ws.wait_limit_ns,
        )
        return out

    def check(self, sync: bool = True) -> None:
        self.ws.check(sync)
        self.ws.check_canaries()

    def close(self, collective: bool = False) -> None:
        self.engine = None
        self.ws.close(collective)


# --------------------------------------------------------------------------------------
# entry point
# --------------------------------------------------------------------------------------

_LAYERS: Dict[tuple, MoEAllToAll] = {}


def get_layer(cfg: MoEConfig, rank: int, world_size: int, group=None, mode: Optional[str] = None) -> MoEAllToAll:
    """Workspace creation is collective and costs milliseconds, so layers are cached per
    configuration; the reference rebuilds its helper object on every call
    (all2all/hipv8.py:379) because it owns no persistent state."""
    key = (cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim, cfg.max_num_tokens, cfg.in_dtype, cfg.out_dtype,
           rank, world_size, id(group), mode)
    layer = _LAYERS.get(key)
    if layer is None:
        resolved = mode or default_mode()
        full = key[:-1] + (resolved, torch.cuda.current_device())
        layer = _LAYERS.get(full)
        if layer is None:
            layer = MoEAllToAll(cfg, rank, world_size, group, mode=resolved)
            _LAYERS[full] = layer
        if torch.cuda.device_count() == 1 or world_size > 1:
            _LAYERS[key] = layer  # short key: one device per process, so the device need not be part of it
    return layer


def release_layers() -> None:
    """Free every cached workspace (collective: all ranks must call it while idle)."""
    for layer in {id(v): v for v in _LAYERS.values()}.values():
        layer.close(collective=True)
    _LAYERS.clear()


def _cpu_ranks_share_a_node() -> bool:
    from ..parallel.host_symm import single_node

    return single_node()


def custom_kernel(data: MoEInput, backend: str = "auto", mode: Optional[str] = None) -> torch.Tensor:
    """Dispatch -> ``* (1 + rank)`` -> combine; returns ``y[num_tokens, hidden]`` in
    ``cfg.out_dtype`` on the rank's device (all2all/reference.py:256-272).

    ``backend``: "auto" = the fused kernels for CUDA tensors, the shared-memory operators
    (models/host_ops.py) for CPU tensors when all ranks share a machine, library collectives
    otherwise; "shm" and "torch" force the latter two.  ``mode`` picks the protocol ("dedup" or
    "direct"; default on GPUs ``B200_MOE_MODE`` or "dedup", on CPU ranks ``B200_HOST_MOE_MODE`` or
    "direct")."""
    cfg, rank_data, rank, world_size = data
    x = rank_data.x
    if backend == "shm" or (backend == "auto" and not x.is_cuda and _cpu_ranks_share_a_node()):
        from . import host_ops

        return host_ops.moe_custom_kernel(data, mode=mode)
    if backend == "torch" or (backend == "auto" and not x.is_cuda):
        ata = TorchAllToAll(cfg, rank, world_size)
        n_tok, ex, em = ata.dispatch(x, rank_data.indices)
        ey = ex.to(cfg.out_dtype) * (1 + rank)
        y = torch.zeros(cfg.max_num_tokens, cfg.hidden_dim, dtype=cfg.out_dtype, device=x.device)
        ata.combine(y, rank_data.weights, em, ey, n_tok)
        return y[: rank_data.num_tokens]
    layer = get_layer(cfg, rank, world_size, mode=mode)
    return layer.forward(x, rank_data.indices, rank_data.weights, 1 + rank)
