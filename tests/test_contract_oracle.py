"""CPU tests of the contracts, shape lists and communication-free oracles."""
import torch

from amd_distributed_2025_b200 import contract, oracle
from amd_distributed_2025_b200.contract import MoEConfig, RankTestData


def _data(cfg, ws, seed=3, **kw):
    out = []
    for r in range(ws):
        g = torch.Generator(device="cpu")
        g.manual_seed(seed + r)
        out.append(RankTestData(cfg, g, r, device="cpu", **kw))
    return out


def test_shape_lists_match_task_files():
    a2a = contract.load_task("all2all")
    assert len(a2a["tests"]) == 9 and len(a2a["benchmarks"]) == 5 and len(a2a["speed_of_light"]) == 5
    assert all(s["world_size"] == 8 for s in a2a["tests"] + a2a["benchmarks"])
    grs = contract.load_task("gemm_rs")
    assert len(grs["tests"]) == 11 and len(grs["benchmarks"]) == 6 and len(grs["speed_of_light"]) == 6
    assert grs["tests"][0] == {"world_size": 8, "m": 64, "n": 2880, "k": 2880, "has_bias": True, "seed": 2035}
    assert a2a["checker"] == {"rtol": 1e-2, "atol": 5e-3}
    assert grs["checker"] == {"rtol": 1e-2, "atol": 1e-2}


def test_reference_style_generator_properties():
    cfg, d, rank, ws = contract.generate_moe_input(64, 6, 128, 32, seed=5, rank=1, world_size=8, device="cpu")
    assert cfg.in_dtype == torch.float16 and cfg.out_dtype == torch.float16
    assert 1 <= d.num_tokens < 32
    assert d.indices.dtype == torch.int32 and d.indices.shape == (d.num_tokens, 6)
    assert d.weights.dtype == torch.float32 and float(d.weights.min()) >= 0 and float(d.weights.max()) < 1
    assert d.x.dtype == torch.float16 and d.x.shape == (d.num_tokens, 128)
    # experts of one token are distinct
    for row in d.indices.tolist():
        assert len(set(row)) == 6 and all(0 <= e < 64 for e in row)
    # seeded: same call, same data
    _, d2, _, _ = contract.generate_moe_input(64, 6, 128, 32, seed=5, rank=1, world_size=8, device="cpu")
    assert torch.equal(d.x, d2.x) and torch.equal(d.indices, d2.indices)


def test_benchmark_factory_variants():
    cfg, d, _, _ = contract.make_moe_inputs(64, 6, 64, 512, 7, 0, 8, device="cpu", dtype=torch.bfloat16,
                                           fixed_num_tokens=512, routing="zipf", weights="softmax")
    assert d.num_tokens == 512 and d.x.dtype == torch.bfloat16
    assert torch.allclose(d.weights.sum(1), torch.ones(512), atol=1e-5)
    for row in d.indices.tolist():
        assert len(set(row)) == 6
    # Zipf routing is skewed towards low expert ids
    counts = torch.bincount(d.indices.reshape(-1).long(), minlength=64)
    assert counts[:8].sum() > 3 * counts[-8:].sum()


def test_gemm_rs_generators():
    a, w, b = contract.generate_gemm_rs_input(2, 8, 64, 48, 256, True, 11, device="cpu")
    assert a.shape == (64, 32) and w.shape == (48, 32) and b.shape == (48,)
    assert a.dtype == torch.bfloat16 and float(a.abs().max()) <= 0.0101
    _, _, b2 = contract.generate_gemm_rs_input(5, 8, 64, 48, 256, True, 11, device="cpu")
    assert torch.equal(b, b2)  # bias generator is re-seeded with the seed alone: same on all ranks
    a3, _, none = contract.make_gemm_rs_inputs(0, 2, 64, 48, 256, False, 11, device="cpu")
    assert none is None and a3.float().std() > 0.5


def test_dispatch_oracle_order_and_owner_map():
    cfg = MoEConfig(8, 2, 16, 4, torch.float32, torch.float32)
    ws = 2
    data = _data(cfg, ws, fixed_num_tokens=4)
    for r in range(ws):
        n, x, meta = oracle.moe_dispatch_oracle(cfg, data, r)
        e_local = 4
        assert int(n.sum()) == sum(int(((d.indices // e_local) == r).sum()) for d in data)
        for e in range(e_local):
            rows = meta[e, : int(n[e])]
            assert torch.all(rows[:, 0] == r * e_local + e)  # owner = e // E_local, local id = e % E_local
            keys = [(int(a), int(b), int(c)) for a, b, c in rows[:, 1:4].tolist()]
            assert keys == sorted(keys)  # (src_rank, src_token, src_k) ascending
            for j, (s, t, k) in enumerate(keys):
                assert int(data[s].indices[t, k]) == r * e_local + e
                assert torch.equal(x[e, j], data[s].x[t])


def test_expected_output_scale_is_per_owner_rank():
    cfg = MoEConfig(8, 2, 8, 4, torch.float32, torch.float32)
    g = torch.Generator().manual_seed(0)
    d = RankTestData(cfg, g, 0, device="cpu", fixed_num_tokens=3)
    y = oracle.moe_expected_output(cfg, d, world_size=4)
    owner = d.indices.long() // 2
    manual = ((1 + owner).float() * d.weights).sum(1, keepdim=True) * d.x
    assert torch.allclose(y, manual, rtol=1e-5, atol=1e-6)


def test_reference_rounding_emulation_close_to_truth_fp16():
    cfg = MoEConfig(64, 6, 256, 16)
    g = torch.Generator().manual_seed(1)
    d = RankTestData(cfg, g, 0, device="cpu", fixed_num_tokens=16)
    truth = oracle.moe_expected_output(cfg, d, 8)
    emu = oracle.moe_expected_output(cfg, d, 8, emulate_reference_rounding=True)
    ok, msg = oracle.check_moe_output(truth, emu)
    assert ok, msg


def test_gemm_rs_truth_counts_bias_world_size_times():
    ws, m, n, k = 4, 16, 8, 64
    ins = [contract.make_gemm_rs_inputs(r, ws, m, n, k, True, 3, device="cpu") for r in range(ws)]
    a = [i[0] for i in ins]
    w = [i[1] for i in ins]
    bias = ins[0][2]
    full = sum(x.double() @ y.double().T for x, y in zip(a, w))
    for r in range(ws):
        t = oracle.gemm_rs_truth(a, w, bias, r)
        assert torch.allclose(t, full[r * 4 : (r + 1) * 4] + ws * bias.double())
        t1 = oracle.gemm_rs_truth(a, w, bias, r, bias_mode="once")
        assert torch.allclose(t1, full[r * 4 : (r + 1) * 4] + bias.double())
    ref = oracle.gemm_rs_reference_rounding(a, w, bias, 0)
    ok, msg = oracle.check_gemm_rs_output(ref, oracle.gemm_rs_truth(a, w, bias, 0).to(torch.bfloat16))
    assert ok, msg


def test_checkers_reject_wrong_results():
    exp = torch.ones(4, 4, dtype=torch.float16)
    assert oracle.check_moe_output(exp.clone(), exp)[0]
    assert not oracle.check_moe_output(exp * 1.05, exp)[0]
    assert not oracle.check_moe_output(exp[:2], exp)[0]
    assert not oracle.check_gemm_rs_output(exp.bfloat16() + 0.5, exp.bfloat16())[0]
