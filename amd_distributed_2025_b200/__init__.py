"""B200-native distributed kernels: MoE expert-parallel dispatch/combine and row-parallel
GEMM fused with reduce-scatter, with the task contracts of the reference
(all2all/task.py:8, gemm-rs/task.py:4).

Public entry points
-------------------
``amd_distributed_2025_b200.models.moe_all2all.custom_kernel(data)``
``amd_distributed_2025_b200.models.gemm_rs.custom_kernel(data)``
``amd_distributed_2025_b200.contract`` -- configs, input generators, shape lists
``amd_distributed_2025_b200.oracle`` -- communication-free ground truth and checkers
``amd_distributed_2025_b200.harness.eval`` -- multi-rank test / benchmark runner
"""
from .contract import (  # noqa: F401
    META_DIM,
    MoEConfig,
    RankTestData,
    generate_gemm_rs_input,
    generate_moe_input,
    make_gemm_rs_inputs,
    make_moe_inputs,
    task_specs,
)

__version__ = "0.1.0"
