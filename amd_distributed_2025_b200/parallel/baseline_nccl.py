"""torch.distributed baselines (NCCL on GPUs, gloo on CPU).

These are the *baseline*, not the product: the same two capabilities expressed with
library collectives.  They serve three purposes: the CPU/gloo path of the framework
(fp32 configuration on two CPU ranks), the comparison arm of the benchmarks on B200,
and an independent cross-check of the fused kernels.

``TorchAllToAll`` keeps the reference class's interface (all2all/reference.py:55-234:
``dispatch(dp_x, indices) -> (expert_num_tokens, expert_x, expert_meta)`` and
``combine(out_tokens, weights, expert_meta, expert_y, expert_num_tokens)``), but has no
per-row Python: routing is a stable sort by destination, the three exchanges are
``all_to_all_single`` calls (counts, rows, metadata -- all2all/reference.py:91,107-119)
and the receive side is one indexed scatter.  The row order inside every expert equals
the reference's.

``gemm_rs_torch`` is the reference GEMM-RS verbatim in behaviour
(gemm-rs/reference.py:52-59): library GEMM, bias add, ``reduce_scatter_tensor``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..contract import META_DIM, MoEConfig, MoEInput, GemmRsInput


class TorchAllToAll:
    META_DIM = META_DIM

    def __init__(self, cfg: MoEConfig, rank: int, world_size: int, group=None):
        self.cfg = cfg
        self.rank = rank
        self.world_size = world_size
        self.group = group
        self.num_local_experts = cfg.num_local_experts(world_size)
        self.max_recv = cfg.max_recv(world_size)

    # -- helpers ---------------------------------------------------------------------
    def _exchange(self, rows: torch.Tensor, meta: torch.Tensor, send_counts: torch.Tensor):
        """Counts, payload and metadata exchange; returns ``(recv_rows, recv_meta)``."""
        ws = self.world_size
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        send_l = send_counts.tolist()
        recv_l = recv_counts.tolist()
        total = sum(recv_l)
        recv_rows = rows.new_empty((total, rows.shape[1]))
        recv_meta = meta.new_empty((total, META_DIM))
        dist.all_to_all_single(recv_rows, rows, recv_l, send_l, group=self.group)
        dist.all_to_all_single(
            recv_meta.view(-1),
            meta.reshape(-1),
            [c * META_DIM for c in recv_l],
            [c * META_DIM for c in send_l],
            group=self.group,
        )
        return recv_rows, recv_meta

    # -- dispatch --------------------------------------------------------------------
    def dispatch(self, dp_x: torch.Tensor, indices: torch.Tensor):
        cfg, ws, dev = self.cfg, self.world_size, dp_x.device
        k = indices.shape[1]
        flat = indices.reshape(-1).to(torch.int64)
        dst = flat // self.num_local_experts
        order = torch.argsort(dst, stable=True)  # grouped by destination, (t, k) order kept
        send_counts = torch.bincount(dst, minlength=ws)
        tok = order // k
        meta = torch.stack(
            [flat[order], torch.full_like(order, self.rank), tok, order % k, torch.zeros_like(order)], dim=1
        ).to(torch.int32)
        recv_rows, recv_meta = self._exchange(dp_x[tok].contiguous(), meta.contiguous(), send_counts)

        local_e = recv_meta[:, 0].to(torch.int64) % self.num_local_experts
        order2 = torch.argsort(local_e, stable=True)
        counts = torch.bincount(local_e, minlength=self.num_local_experts)
        starts = torch.cumsum(counts, 0) - counts
        sorted_e = local_e[order2]
        pos = torch.arange(order2.numel(), device=dev) - starts[sorted_e]
        expert_x = torch.empty(
            (self.num_local_experts, self.max_recv, cfg.hidden_dim), dtype=cfg.in_dtype, device=dev
        )
        expert_meta = torch.empty(
            (self.num_local_experts, self.max_recv, META_DIM), dtype=torch.int32, device=dev
        )
        expert_x[sorted_e, pos] = recv_rows[order2]
        expert_meta[sorted_e, pos] = recv_meta[order2]
        return counts.to(torch.int32), expert_x, expert_meta

    # -- combine ---------------------------------------------------------------------
    def combine(
        self,
        out_tokens: torch.Tensor,
        weights: torch.Tensor,
        expert_meta: torch.Tensor,
        expert_y: torch.Tensor,
        expert_num_tokens: torch.Tensor,
    ) -> torch.Tensor:
        cfg, ws, dev = self.cfg, self.world_size, out_tokens.device
        pos = torch.arange(self.max_recv, device=dev)
        valid = pos[None, :] < expert_num_tokens.to(torch.int64)[:, None]  # [E_local, max_recv]
        rows = expert_y[valid]  # (expert, slot) order
        meta = expert_meta[valid]
        dst = meta[:, 1].to(torch.int64)
        order = torch.argsort(dst, stable=True)
        send_counts = torch.bincount(dst, minlength=ws)
        recv_rows, recv_meta = self._exchange(rows[order].contiguous(), meta[order].contiguous(), send_counts)
        src_token = recv_meta[:, 2].to(torch.int64)
        src_k = recv_meta[:, 3].to(torch.int64)
        w = weights[src_token, src_k].to(torch.float32)
        acc = out_tokens.to(torch.float32)
        t, k = weights.shape
        if recv_rows.shape[0] == t * k:
            # every (token, k) entry came back exactly once: order the rows by (token, k) and
            # sum over k in that fixed order (deterministic, and no scatter)
            order = torch.argsort(src_token * k + src_k)
            contrib = (recv_rows[order].to(torch.float32) * w[order][:, None]).view(t, k, -1)
            acc[:t] += contrib.sum(dim=1)
        else:
            acc.index_add_(0, src_token, recv_rows.to(torch.float32) * w[:, None])
        out_tokens.copy_(acc)
        return out_tokens


def moe_torch(data: MoEInput, group=None) -> torch.Tensor:
    """Dispatch -> per-rank scale -> combine with library collectives
    (driver shape of all2all/reference.py:256-272)."""
    cfg, rank_data, rank, world_size = data
    ata = TorchAllToAll(cfg, rank, world_size, group)
    expert_num, expert_x, expert_meta = ata.dispatch(rank_data.x, rank_data.indices)
    expert_y = expert_x.to(cfg.out_dtype) * (1 + rank)
    y = torch.zeros(cfg.max_num_tokens, cfg.hidden_dim, dtype=cfg.out_dtype, device=rank_data.x.device)
    ata.combine(y, rank_data.weights, expert_meta, expert_y, expert_num)
    return y[: rank_data.num_tokens]


def gemm_rs_torch(data: GemmRsInput, group=None) -> torch.Tensor:
    """Library GEMM + bias + reduce-scatter (gemm-rs/reference.py:52-59).

    On backends without ``reduce_scatter_tensor`` (gloo) an all-reduce followed by a
    slice stands in; results are identical up to summation order.
    """
    a, w, bias = data
    ws = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    out = torch.matmul(a, w.T)
    if bias is not None:
        out = out + bias
    rows = a.shape[0] // ws
    if ws == 1:
        return out
    if a.is_cuda:
        rs = torch.empty((rows, w.shape[0]), dtype=out.dtype, device=a.device)
        dist.reduce_scatter_tensor(rs, out, group=group)
        return rs
    # gloo has no bf16 reduction on every build: reduce in fp32, round back.
    full = out.to(torch.float32)
    dist.all_reduce(full, group=group)
    return full[rank * rows : (rank + 1) * rows].to(out.dtype).contiguous()
