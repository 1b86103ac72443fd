"""Task contracts: configuration objects, per-rank input generators and shape lists.

Two capabilities share this module.

* MoE expert-parallel dispatch/combine.  The input of ``custom_kernel`` is the 4-tuple
  ``(MoEConfig, RankTestData, rank, world_size)`` (reference: all2all/task.py:8,
  all2all/reference.py:237-253).  ``RankTestData`` carries ``num_tokens``,
  ``indices[T, k] int32``, ``weights[T, k] fp32`` and ``x[T, H]``
  (all2all/reference.py:20-51).
* Row-parallel GEMM + reduce-scatter.  The input is the 3-tuple
  ``(input[M, K/ws], weight[N, K/ws], bias[N] | None)`` in bf16
  (gemm-rs/task.py:4, gemm-rs/reference.py:5-33).

``generate_moe_input`` / ``generate_gemm_rs_input`` draw from a torch generator with
the same sequence of calls as the reference generators, so that on a CUDA device the
same seed yields the same tensors.  ``make_moe_inputs`` / ``make_gemm_rs_inputs`` are
the wider factories used by the benchmark configurations (fixed token counts, Zipf
routing, softmax weights, normal-distributed GEMM operands, any device).
"""
from __future__ import annotations

import dataclasses
import os
from typing import Any, Dict, List, Optional, Tuple

import torch

META_DIM = 5  # (global_expert, src_rank, src_token, src_k, pad) -- all2all/reference.py:56


@dataclasses.dataclass
class MoEConfig:
    """Hyper-parameters of one MoE dispatch/combine problem (all2all/reference.py:10-17)."""

    num_experts: int
    experts_per_token: int
    hidden_dim: int
    max_num_tokens: int
    in_dtype: torch.dtype = torch.float16
    out_dtype: torch.dtype = torch.float16

    def num_local_experts(self, world_size: int) -> int:
        if self.num_experts % world_size:
            raise ValueError(
                f"num_experts={self.num_experts} is not divisible by world_size={world_size}"
            )
        return self.num_experts // world_size

    def max_recv(self, world_size: int) -> int:
        """Rows reserved per local expert: every token of every rank may pick it."""
        return self.max_num_tokens * world_size


class RankTestData:
    """Tokens, routing and routing weights owned by one data-parallel rank.

    ``RankTestData(cfg, rng, rank)`` reproduces the reference constructor
    (all2all/reference.py:21-51): a random token count in ``[1, max_num_tokens)``, per
    token the first ``k`` entries of a random permutation of the experts, uniform
    ``[0, 1)`` fp32 weights and standard-normal activations.  The extra keyword
    arguments select the benchmark variants and default to the reference behaviour.
    """

    def __init__(
        self,
        cfg: MoEConfig,
        rng: torch.Generator,
        rank: int,
        *,
        device: Optional[torch.device] = None,
        fixed_num_tokens: Optional[int] = None,
        routing: str = "uniform",
        weights: str = "rand",
        zipf_s: float = 1.2,
    ):
        if device is None:
            device = torch.device(f"cuda:{rank}")
        device = torch.device(device)
        k = cfg.experts_per_token
        if fixed_num_tokens is None:
            hi = max(cfg.max_num_tokens, 2)
            self.num_tokens = int(torch.randint(1, hi, [1], generator=rng, device=device).item())
        else:
            if not 0 <= fixed_num_tokens <= cfg.max_num_tokens:
                raise ValueError("fixed_num_tokens must lie in [0, max_num_tokens]")
            self.num_tokens = int(fixed_num_tokens)
        t = self.num_tokens

        if routing == "uniform" and fixed_num_tokens is None:
            # Same call sequence as the reference: one randperm per token.
            self.indices = torch.empty(t, k, dtype=torch.int32, device=device)
            for i in range(t):
                perm = torch.randperm(cfg.num_experts, generator=rng, device=device)
                self.indices[i] = perm[:k]
        elif routing == "uniform":
            # Distinct experts per token, drawn in one batched call (Gumbel top-k with
            # flat logits is a uniform sample without replacement).
            noise = torch.rand(t, cfg.num_experts, generator=rng, device=device)
            self.indices = noise.topk(k, dim=1).indices.to(torch.int32)
        elif routing == "zipf":
            # Sampling without replacement from p(e) ~ 1/(e+1)^s via Gumbel top-k.
            ranks = torch.arange(1, cfg.num_experts + 1, device=device, dtype=torch.float32)
            logp = -zipf_s * ranks.log()
            u = torch.rand(t, cfg.num_experts, generator=rng, device=device).clamp_(1e-12, 1 - 1e-7)
            gumbel = -(-u.log()).log()
            self.indices = (logp + gumbel).topk(k, dim=1).indices.to(torch.int32)
        else:
            raise ValueError(f"unknown routing {routing!r}")

        if weights == "rand":
            self.weights = torch.rand(t, k, dtype=torch.float32, generator=rng, device=device)
        elif weights == "softmax":
            logits = torch.randn(t, k, dtype=torch.float32, generator=rng, device=device)
            self.weights = torch.softmax(logits, dim=1)
        else:
            raise ValueError(f"unknown weights {weights!r}")

        self.x = torch.randn(t, cfg.hidden_dim, dtype=cfg.in_dtype, generator=rng, device=device)

    def to(self, device) -> "RankTestData":
        out = object.__new__(RankTestData)
        out.num_tokens = self.num_tokens
        out.indices = self.indices.to(device)
        out.weights = self.weights.to(device)
        out.x = self.x.to(device)
        return out


MoEInput = Tuple[MoEConfig, RankTestData, int, int]
GemmRsInput = Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]


def generate_moe_input(
    num_experts: int,
    experts_per_token: int,
    hidden_dim: int,
    max_num_tokens: int,
    seed: int,
    rank: int,
    world_size: int,
    device: Optional[torch.device] = None,
) -> MoEInput:
    """Reference-compatible MoE input factory (all2all/reference.py:237-253).

    fp16 in and out, generator seeded with ``seed + rank`` on the rank's device.
    """
    device = torch.device(f"cuda:{rank}") if device is None else torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + rank)
    cfg = MoEConfig(
        num_experts=num_experts,
        experts_per_token=experts_per_token,
        hidden_dim=hidden_dim,
        max_num_tokens=max_num_tokens,
        in_dtype=torch.float16,
        out_dtype=torch.float16,
    )
    return cfg, RankTestData(cfg, gen, rank, device=device), rank, world_size


def make_moe_inputs(
    num_experts: int,
    experts_per_token: int,
    hidden_dim: int,
    max_num_tokens: int,
    seed: int,
    rank: int,
    world_size: int,
    *,
    device: Optional[torch.device] = None,
    dtype: torch.dtype = torch.float16,
    fixed_num_tokens: Optional[int] = None,
    routing: str = "uniform",
    weights: str = "rand",
    zipf_s: float = 1.2,
) -> MoEInput:
    """Benchmark-oriented MoE input factory; returns the same 4-tuple as the reference."""
    device = torch.device(f"cuda:{rank}") if device is None else torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + rank)
    cfg = MoEConfig(num_experts, experts_per_token, hidden_dim, max_num_tokens, dtype, dtype)
    data = RankTestData(
        cfg,
        gen,
        rank,
        device=device,
        fixed_num_tokens=fixed_num_tokens,
        routing=routing,
        weights=weights,
        zipf_s=zipf_s,
    )
    return cfg, data, rank, world_size


def generate_gemm_rs_input(
    rank: int,
    world_size: int,
    m: int,
    n: int,
    k: int,
    has_bias: bool,
    seed: int,
    device: Optional[torch.device] = None,
) -> GemmRsInput:
    """Reference-compatible GEMM-RS input factory (gemm-rs/reference.py:5-33).

    Operands are uniform in ``[-0.01, 0.01]`` bf16; the bias generator is re-seeded with
    ``seed`` alone, so every rank holds the same bias.
    """
    device = torch.device(f"cuda:{rank}") if device is None else torch.device(device)
    if m % world_size or k % world_size:
        raise ValueError("m and k must be divisible by world_size")
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + rank)
    local_k = k // world_size

    def unit(shape):
        return (torch.rand(shape, dtype=torch.bfloat16, device=device, generator=gen) * 2 - 1) * 0.01

    a = unit((m, local_k))
    w = unit((n, local_k))
    bias = None
    if has_bias:
        gen.manual_seed(seed)
        bias = unit((n,))
    return a, w, bias


def make_gemm_rs_inputs(
    rank: int,
    world_size: int,
    m: int,
    n: int,
    k: int,
    has_bias: bool,
    seed: int,
    *,
    device: Optional[torch.device] = None,
    dist: str = "normal",
    a_std: float = 1.0,
    w_std: float = 0.02,
    bias_std: float = 0.02,
) -> GemmRsInput:
    """GEMM-RS inputs for the benchmark configurations: A ~ N(0,1), W, bias ~ N(0,0.02)."""
    if dist == "reference":
        return generate_gemm_rs_input(rank, world_size, m, n, k, has_bias, seed, device)
    device = torch.device(f"cuda:{rank}") if device is None else torch.device(device)
    if m % world_size or k % world_size:
        raise ValueError("m and k must be divisible by world_size")
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + rank)
    local_k = k // world_size
    a = (torch.randn((m, local_k), dtype=torch.float32, device=device, generator=gen) * a_std).to(torch.bfloat16)
    w = (torch.randn((n, local_k), dtype=torch.float32, device=device, generator=gen) * w_std).to(torch.bfloat16)
    bias = None
    if has_bias:
        gen.manual_seed(seed)
        bias = (torch.randn((n,), dtype=torch.float32, device=device, generator=gen) * bias_std).to(torch.bfloat16)
    return a, w, bias


# --------------------------------------------------------------------------------------
# Shape lists (configs/*.yml)
# --------------------------------------------------------------------------------------

_CONFIG_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "configs")


def load_task(name: str) -> Dict[str, Any]:
    """Load ``configs/<name>.yml``: ``tests``, ``benchmarks``, ``speed_of_light`` lists and metadata."""
    import yaml

    path = os.path.join(_CONFIG_DIR, f"{name}.yml")
    with open(path, "r", encoding="utf-8") as fh:
        return yaml.safe_load(fh)


def task_specs(name: str, section: str) -> List[Dict[str, Any]]:
    """Return the list of shape dictionaries of ``section`` ("tests" or "benchmarks")."""
    return list(load_task(name)[section])
