"""Communication-free oracles and checkers for both tasks.

The reference checks a solution against a torch.distributed implementation
(all2all/reference.py:256-283, gemm-rs/reference.py:36-71).  This module states the
same mathematics *without* collectives: given the inputs of **all** ranks it computes,
for one rank, the exact dispatch layouts and the combined output (MoE), or the
reduce-scattered slice (GEMM-RS).  Tests use it as ground truth on CPU and GPU; the
distributed NCCL/gloo restatement lives in ``parallel/baseline_nccl.py``.

Facts encoded here (and pinned by unit tests):

* expert ``e`` lives on rank ``e // E_local`` as local expert ``e % E_local``
  (all2all/reference.py:81,142);
* inside a local expert, rows are ordered by ``(src_rank, src_token, src_k)``: the send
  lists are built in ``(t, k)`` order per destination (all2all/reference.py:79-86), the
  exchange concatenates by source rank (all2all/reference.py:107-112) and rows are
  appended in arrival order (all2all/reference.py:140-146);
* the expert op is a per-*rank* scale ``(1 + owner_rank)`` rounded to ``out_dtype``
  (all2all/reference.py:262);
* the reference combine accumulates in ``out_dtype``, one rounding per addend, in
  arrival order = ascending global expert id (all2all/reference.py:226-232);
* GEMM-RS adds the bias on every rank before the reduction, so the checker expects
  ``sum_r A_r W_r^T + world_size * bias`` (gemm-rs/reference.py:54-59).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from .contract import META_DIM, MoEConfig, RankTestData

MOE_RTOL, MOE_ATOL = 1e-2, 5e-3  # all2all/reference.py:279
GEMM_RS_RTOL, GEMM_RS_ATOL = 1e-2, 1e-2  # gemm-rs/reference.py:67


# --------------------------------------------------------------------------------------
# MoE
# --------------------------------------------------------------------------------------

def moe_dispatch_oracle(
    cfg: MoEConfig, all_data: Sequence[RankTestData], rank: int
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Expected ``(expert_num_tokens, expert_x, expert_meta)`` on ``rank``.

    Rows past ``expert_num_tokens[e]`` are zero here (the reference leaves them
    uninitialised); compare valid rows only.
    """
    ws = len(all_data)
    e_local = cfg.num_local_experts(ws)
    max_recv = cfg.max_recv(ws)
    device = all_data[rank].x.device
    xs, metas = [], []
    for src, d in enumerate(all_data):
        k = d.indices.shape[1]
        flat = d.indices.reshape(-1).to(torch.int64).to(device)
        mine = torch.nonzero((flat // e_local) == rank).reshape(-1)  # ascending = (t, k) order
        tok = mine // k
        meta = torch.stack(
            [flat[mine], torch.full_like(mine, src), tok, mine % k, torch.zeros_like(mine)], dim=1
        )
        xs.append(d.x.to(device)[tok])
        metas.append(meta)
    x_all = torch.cat(xs, 0)
    meta_all = torch.cat(metas, 0)
    local_e = meta_all[:, 0] % e_local
    order = torch.argsort(local_e, stable=True)
    counts = torch.bincount(local_e, minlength=e_local)
    starts = torch.cumsum(counts, 0) - counts
    sorted_e = local_e[order]
    pos = torch.arange(order.numel(), device=device) - starts[sorted_e]
    expert_x = torch.zeros(e_local, max_recv, cfg.hidden_dim, dtype=cfg.in_dtype, device=device)
    expert_meta = torch.zeros(e_local, max_recv, META_DIM, dtype=torch.int32, device=device)
    expert_x[sorted_e, pos] = x_all[order]
    expert_meta[sorted_e, pos] = meta_all[order].to(torch.int32)
    return counts.to(torch.int32), expert_x, expert_meta


def moe_expected_output(
    cfg: MoEConfig,
    data: RankTestData,
    world_size: int,
    *,
    emulate_reference_rounding: bool = False,
    acc_dtype: torch.dtype = torch.float64,
) -> torch.Tensor:
    """Expected combined output of one rank, ``[num_tokens, hidden]`` in ``out_dtype``.

    Only the rank's own tokens matter: every expert row is ``x[t]`` scaled by
    ``1 + owner(e)``.  With ``emulate_reference_rounding`` the sum follows the
    reference's rounding points (addend rounded to ``out_dtype``, accumulator rounded
    after every add, ascending expert order); otherwise it is accumulated in
    ``acc_dtype`` and rounded once.
    """
    e_local = cfg.num_local_experts(world_size)
    idx = data.indices.to(torch.int64)
    owner = idx // e_local  # [T, k]
    scale = (1 + owner).to(torch.float32)
    x = data.x
    t, k = idx.shape
    if emulate_reference_rounding:
        order = torch.argsort(idx, dim=1)
        acc = torch.zeros(t, cfg.hidden_dim, dtype=cfg.out_dtype, device=x.device)
        for j in range(k):
            col = order[:, j]
            s = scale.gather(1, col[:, None])  # [T, 1]
            w = data.weights.gather(1, col[:, None]).to(torch.float32)
            y = (x.to(cfg.out_dtype) * s.to(cfg.out_dtype)).to(cfg.out_dtype)
            acc = (acc.to(torch.float32) + y.to(torch.float32) * w).to(cfg.out_dtype)
        return acc
    acc = torch.zeros(t, cfg.hidden_dim, dtype=acc_dtype, device=x.device)
    for j in range(k):
        y = (x.to(cfg.out_dtype) * scale[:, j : j + 1].to(cfg.out_dtype)).to(cfg.out_dtype)
        acc += y.to(acc_dtype) * data.weights[:, j : j + 1].to(acc_dtype)
    return acc.to(cfg.out_dtype)


def check_moe_output(
    output: torch.Tensor, expected: torch.Tensor, rtol: float = MOE_RTOL, atol: float = MOE_ATOL
) -> Tuple[bool, str]:
    """Reference acceptance test: same device and ``allclose(rtol=1e-2, atol=5e-3)``
    (all2all/reference.py:275-283)."""
    if output.device != expected.device:
        return False, f"Output device mismatch: {output.device} != {expected.device}"
    if output.shape != expected.shape:
        return False, f"Output shape mismatch: {tuple(output.shape)} != {tuple(expected.shape)}"
    if not torch.allclose(output.to(expected.dtype), expected, rtol=rtol, atol=atol):
        err = (output.float() - expected.float()).abs().max().item()
        return False, f"Output values mismatch, max abs err {err:.4g}"
    return True, ""


def compare_dispatch_layout(
    got: Tuple[torch.Tensor, torch.Tensor, torch.Tensor],
    want: Tuple[torch.Tensor, torch.Tensor, torch.Tensor],
    *,
    ordered: bool = True,
) -> Tuple[bool, str]:
    """Compare the valid rows of two dispatch results.

    ``ordered=True`` demands the reference row order; otherwise rows of one expert are
    compared as a multiset keyed by ``(src_rank, src_token, src_k)``.
    """
    n_got, x_got, m_got = got
    n_want, x_want, m_want = want
    if not torch.equal(n_got.to(torch.int64).cpu(), n_want.to(torch.int64).cpu()):
        return False, f"expert_num_tokens differ: {n_got.tolist()} != {n_want.tolist()}"
    for e, n in enumerate(n_want.tolist()):
        mg, mw = m_got[e, :n].cpu(), m_want[e, :n].cpu()
        xg, xw = x_got[e, :n].cpu(), x_want[e, :n].cpu()
        if not ordered and n:
            def key(m):
                return (m[:, 1].to(torch.int64) << 40) + (m[:, 2].to(torch.int64) << 8) + m[:, 3].to(torch.int64)

            og, ow = torch.argsort(key(mg)), torch.argsort(key(mw))
            mg, xg, mw, xw = mg[og], xg[og], mw[ow], xw[ow]
        if not torch.equal(mg[:, :4], mw[:, :4]):
            return False, f"expert_meta differs for local expert {e}"
        if not torch.equal(xg, xw):
            return False, f"expert_x differs for local expert {e}"
    return True, ""


# --------------------------------------------------------------------------------------
# GEMM + reduce-scatter
# --------------------------------------------------------------------------------------

def gemm_rs_truth(
    inputs: Sequence[torch.Tensor],
    weights: Sequence[torch.Tensor],
    bias: Optional[torch.Tensor],
    rank: int,
    *,
    bias_mode: str = "per_rank",
    dtype: torch.dtype = torch.float64,
) -> torch.Tensor:
    """``[M/ws, N]`` slice of ``sum_r A_r W_r^T (+ bias)`` for ``rank``, in ``dtype`` (no rounding).

    ``bias_mode="per_rank"`` adds ``world_size * bias`` (what the reference checker
    expects), ``"once"`` adds ``bias``.
    """
    ws = len(inputs)
    m = inputs[0].shape[0]
    rows = m // ws
    sl = slice(rank * rows, (rank + 1) * rows)
    acc = None
    for a, w in zip(inputs, weights):
        part = a[sl].to(dtype) @ w.to(dtype).T
        acc = part if acc is None else acc + part
    if bias is not None:
        factor = ws if bias_mode == "per_rank" else 1
        acc = acc + factor * bias.to(dtype)
    return acc


def gemm_rs_reference_rounding(
    inputs: Sequence[torch.Tensor],
    weights: Sequence[torch.Tensor],
    bias: Optional[torch.Tensor],
    rank: int,
) -> torch.Tensor:
    """The reference's rounding points: bf16 matmul result, bf16 bias add on every rank,
    bf16 sum over ranks in rank order (gemm-rs/reference.py:54-59)."""
    ws = len(inputs)
    rows = inputs[0].shape[0] // ws
    sl = slice(rank * rows, (rank + 1) * rows)
    acc = None
    for a, w in zip(inputs, weights):
        part = (a[sl].to(torch.float32) @ w.to(torch.float32).T).to(torch.bfloat16)
        if bias is not None:
            part = part + bias
        acc = part if acc is None else (acc + part)
    return acc


def gemm_rs_fused_rounding(
    inputs: Sequence[torch.Tensor],
    weights: Sequence[torch.Tensor],
    bias: Optional[torch.Tensor],
    rank: int,
    *,
    bias_mode: str = "per_rank",
) -> torch.Tensor:
    """The fused kernel's rounding points.  Every rank's partial is rounded to bf16 (as the
    reference's matmul output is); with ``bias_mode="per_rank"`` the bf16 bias is added to
    it and the sum rounded again, exactly as the reference does on every rank; the
    partials are then summed in fp32 in rank order and rounded once (``"once"`` adds the
    bias to that fp32 sum instead)."""
    ws = len(inputs)
    rows = inputs[0].shape[0] // ws
    sl = slice(rank * rows, (rank + 1) * rows)
    acc = None
    for a, w in zip(inputs, weights):
        part = (a[sl].to(torch.float32) @ w.to(torch.float32).T).to(torch.bfloat16)
        if bias is not None and bias_mode == "per_rank":
            part = part + bias
        part = part.to(torch.float32)
        acc = part if acc is None else acc + part
    if bias is not None and bias_mode != "per_rank":
        acc = acc + bias.to(torch.float32)
    return acc.to(torch.bfloat16)


def check_gemm_rs_output(
    output: torch.Tensor, expected: torch.Tensor, rtol: float = GEMM_RS_RTOL, atol: float = GEMM_RS_ATOL
) -> Tuple[bool, str]:
    """Reference acceptance test: same device and ``allclose(rtol=1e-2, atol=1e-2)``
    (gemm-rs/reference.py:63-71)."""
    if output.device != expected.device:
        return False, f"Output device mismatch: {output.device} != {expected.device}"
    if output.shape != expected.shape:
        return False, f"Output shape mismatch: {tuple(output.shape)} != {tuple(expected.shape)}"
    if not torch.allclose(output.to(expected.dtype), expected, rtol=rtol, atol=atol):
        err = (output.float() - expected.float()).abs().max().item()
        return False, f"Output values mismatch, max abs err {err:.4g}"
    return True, ""


def outlier_fraction(output: torch.Tensor, expected: torch.Tensor, rtol: float, atol: float) -> float:
    """Share of elements outside ``atol + rtol * |expected|``.

    Why a bound on this share replaces a strict ``allclose`` for unit-variance operands: what
    strays is not the rounding of the RESULT (one bf16 ulp never exceeds the task tolerance) but
    the rounding of the PARTIALS.  Every rank's partial has magnitude ~1 whatever the sum is, so
    its bf16 rounding (half an ulp of 2^-8 .. 2^-7) leaves an error of a few 1e-3 in a sum that
    may be near zero, against a tolerance of 1e-2 there; two correct implementations that round
    the partials at different points (fp32 sum of bf16 partials here, a bf16 running sum in the
    library's ring) differ by more than the tolerance on 0.5-1 % of the elements at 8 ranks
    (measured on the CPU: 0.66 % for 512 x 3584 x 14336).  Against a result with the SAME rounding
    points the share must stay below 1e-3."""
    diff = (output.to(torch.float32) - expected.to(torch.float32)).abs()
    tol = atol + rtol * expected.to(torch.float32).abs()
    return float((diff > tol).to(torch.float32).mean())


def relative_error(output: torch.Tensor, truth: torch.Tensor) -> float:
    """Frobenius-norm relative error against an un-rounded truth; the strict check used
    where the reference tolerance is vacuous (outputs far below ``atol``)."""
    num = (output.to(torch.float64) - truth.to(torch.float64)).norm()
    den = truth.to(torch.float64).norm().clamp_min(1e-30)
    return float(num / den)
