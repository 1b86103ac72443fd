"""Multi-process CPU tests (gloo): the library-collective path against the
communication-free oracle, including the exact dispatch row order."""
import torch

from amd_distributed_2025_b200 import contract, oracle
from amd_distributed_2025_b200.harness.eval import run_ranks


def _moe_rank(rank, world_size, spec):
    from amd_distributed_2025_b200.models import moe_all2all
    from amd_distributed_2025_b200.parallel.baseline_nccl import TorchAllToAll

    dev = torch.device("cpu")
    everyone = [
        contract.make_moe_inputs(spec["E"], spec["k"], spec["H"], spec["T"], spec["seed"], r, world_size, device=dev,
                                 dtype=getattr(torch, spec["dtype"]), fixed_num_tokens=spec.get("fixed"),
                                 routing=spec.get("routing", "uniform"), weights=spec.get("weights", "softmax"))
        for r in range(world_size)
    ]
    cfg, mine, _, _ = everyone[rank]
    y = moe_all2all.custom_kernel((cfg, mine, rank, world_size), backend="torch")
    want = oracle.moe_expected_output(cfg, mine, world_size)
    ok, msg = oracle.check_moe_output(y, want)
    rel = oracle.relative_error(y, oracle.moe_expected_output(cfg, mine, world_size))
    # layouts, exact and ordered
    ata = TorchAllToAll(cfg, rank, world_size)
    got = ata.dispatch(mine.x, mine.indices)
    lay_ok, lay_msg = oracle.compare_dispatch_layout(got, oracle.moe_dispatch_oracle(cfg, [e[1] for e in everyone], rank))
    return {"ok": bool(ok), "msg": msg, "rel": rel, "layout_ok": bool(lay_ok), "layout_msg": lay_msg,
            "shape": list(y.shape)}


def test_moe_cpu_fp32_headline_config_two_ranks():
    # 16 experts (8 per rank), top-2, hidden 256, 32 tokens per rank, fp32, softmax weights
    spec = dict(E=16, k=2, H=256, T=32, seed=11, dtype="float32", fixed=32)
    for r in run_ranks(_moe_rank, 2, "gloo", (spec,), 300.0):
        assert r["ok"], r["msg"]
        assert r["layout_ok"], r["layout_msg"]
        assert r["rel"] < 1e-5
        assert r["shape"] == [32, 256]


def test_moe_cpu_fp16_random_token_counts_four_ranks():
    # reference-like: random token counts per rank, some ranks send nothing to some peers
    spec = dict(E=8, k=2, H=64, T=4, seed=1236, dtype="float16", weights="rand")
    for r in run_ranks(_moe_rank, 4, "gloo", (spec,), 300.0):
        assert r["ok"], r["msg"]
        assert r["layout_ok"], r["layout_msg"]


def _gemm_rank(rank, world_size, m, n, k, has_bias):
    from amd_distributed_2025_b200.models import gemm_rs

    everyone = [contract.make_gemm_rs_inputs(r, world_size, m, n, k, has_bias, 5, device="cpu") for r in range(world_size)]
    out = gemm_rs.custom_kernel(everyone[rank], backend="torch")
    truth = oracle.gemm_rs_truth([e[0] for e in everyone], [e[1] for e in everyone], everyone[rank][2], rank)
    ok, msg = oracle.check_gemm_rs_output(out, truth.to(out.dtype))
    return {"ok": bool(ok), "msg": msg, "rel": oracle.relative_error(out, truth), "shape": list(out.shape)}


def test_gemm_rs_cpu_two_ranks_bias_counts_world_size_times():
    for r in run_ranks(_gemm_rank, 2, "gloo", (64, 48, 256, True), 300.0):
        assert r["ok"], r["msg"]
        assert r["rel"] < 1e-2
        assert r["shape"] == [32, 48]


def _reference_arm_rank(rank, world_size):
    from amd_distributed_2025_b200.harness import reference_arm

    ref = reference_arm.load_all2all()
    cfg, mine, _, _ = contract.make_moe_inputs(16, 2, 64, 8, 5, rank, world_size, device="cpu", dtype=torch.float32,
                                               fixed_num_tokens=8, weights="softmax")
    y = ref.ref_kernel(reference_arm.moe_tuple(ref, cfg, mine, rank, world_size))
    ok, msg = oracle.check_moe_output(y, oracle.moe_expected_output(cfg, mine, world_size))
    grs = reference_arm.load_gemm_rs()
    return {"ok": bool(ok), "msg": msg, "has_gemm": hasattr(grs, "ref_kernel") and hasattr(grs, "generate_input")}


def test_unmodified_reference_files_load_and_agree_with_the_oracle():
    """The comparison arm imports the reference's own files (when a copy is present) and its
    result on CPU ranks equals the communication-free oracle."""
    import pytest

    from amd_distributed_2025_b200.harness import reference_arm

    if not reference_arm.reference_available():
        pytest.skip("no copy of the reference files under baseline/_ref")
    for r in run_ranks(_reference_arm_rank, 2, "gloo", (), 300.0):
        assert r["ok"], r["msg"]
        assert r["has_gemm"]
