"""Block-scaled fp8 GEMM: ``c = sum_kb (a_kb @ b_kb.T) * a_scale[:, kb, None] * b_scale[n // 128, kb]``.

The reference tree carries a stand-alone template of this operation that belongs to
neither of its tasks (all2all/hip.py:17-78: inputs ``(a, b, a_scale, b_scale, c)``, fp8
e4m3 operands, fp32 scales per row x 128-wide K block of ``a`` and per 128 x 128 block of
``b``, bf16 result written into ``c``).  The template indexes its operands column-major
(``a[m + k * M]``); this module takes the natural row-major ``a[M, K]`` / ``b[N, K]`` and
accepts the template's layout too, converting it with one transpose copy.  The scale
tensors are read through their strides, so both layouts work without a copy.

The product runs on the fp8 tensor-core path (csrc/fp8_gemm_sm100.cu).  The AMD template
uses the ``e4m3fnuz`` encoding; on NVIDIA hardware the type is ``torch.float8_e4m3fn``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

BLOCK = 128


def fp8_gemm_reference(a: torch.Tensor, b: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor) -> torch.Tensor:
    """Plain PyTorch fp32 statement of the operation (any device)."""
    m, k = a.shape
    n = b.shape[0]
    af, bf = a.to(torch.float32), b.to(torch.float32)
    out = torch.zeros(m, n, dtype=torch.float32, device=a.device)
    nb_index = torch.arange(n, device=a.device) // BLOCK
    for kb in range((k + BLOCK - 1) // BLOCK):
        sl = slice(kb * BLOCK, min((kb + 1) * BLOCK, k))
        part = af[:, sl] @ bf[:, sl].T
        out += part * a_scale[:, kb : kb + 1].to(torch.float32) * b_scale[nb_index, kb][None, :].to(torch.float32)
    return out


def fp8_gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_scale: torch.Tensor,
    b_scale: torch.Tensor,
    c: Optional[torch.Tensor] = None,
    timeout_ms: float = 2000.0,
) -> torch.Tensor:
    """``a [M, K]``, ``b [N, K]`` in ``float8_e4m3fn``; ``a_scale [M, ceil(K/128)]``,
    ``b_scale [ceil(N/128), ceil(K/128)]`` fp32; returns (and fills, if given) bf16 ``c [M, N]``."""
    from . import _ext

    ext = _ext.load()
    if not a.is_contiguous():  # e.g. the template's column-major storage, a [K, M] buffer viewed as [M, K]
        a = a.contiguous()
    if not b.is_contiguous():
        b = b.contiguous()
    if c is None:
        c = torch.empty((a.shape[0], b.shape[0]), dtype=torch.bfloat16, device=a.device)
    flag = torch.zeros(1, dtype=torch.int32, device=a.device)
    ext.fp8_gemm(a, b, a_scale, b_scale, c, flag, int(timeout_ms * 1e6))
    return c


def custom_kernel(data: Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]) -> torch.Tensor:
    """Entry point with the template's 5-tuple ``(a, b, a_scale, b_scale, c)`` (all2all/hip.py:75-78)."""
    a, b, a_scale, b_scale, c = data
    return fp8_gemm(a, b, a_scale, b_scale, c)
