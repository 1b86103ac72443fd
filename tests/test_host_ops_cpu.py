"""CPU ranks over shared memory: the one-sided protocols of the two operators under real
concurrency (2 to 8 processes), against the communication-free oracle."""
import multiprocessing as mp
import os
import time

import pytest
import torch

from amd_distributed_2025_b200 import contract, oracle
from amd_distributed_2025_b200.harness.eval import run_ranks

CPU = torch.device("cpu")


def _patient():
    """Ranks of a loaded test machine may reach a call seconds apart: a long wait limit costs
    nothing when everything works (set before the package reads it at import)."""
    os.environ["B200_WAIT_LIMIT_MS"] = "60000"


def _moe_inputs(spec, seed, world_size):
    return [
        contract.make_moe_inputs(spec["E"], spec["k"], spec["H"], spec["T"], seed, r, world_size, device=CPU,
                                 dtype=getattr(torch, spec["dtype"]), fixed_num_tokens=spec.get("fixed"),
                                 routing=spec.get("routing", "uniform"), weights=spec.get("weights", "softmax"))
        for r in range(world_size)
    ]


def _moe_rank(rank, world_size, spec, calls):
    _patient()
    from amd_distributed_2025_b200.models import host_ops, moe_all2all

    res = {"ok": True, "msg": "", "layout_ok": True, "layout_msg": "", "rel": 0.0}
    for call in range(calls):
        # same configuration, new tokens and routing every call: the buffers are reused with
        # nothing but the protocol's flags between the calls
        everyone = _moe_inputs(spec, spec["seed"] + 17 * call, world_size)
        cfg, mine, _, _ = everyone[rank]
        y = moe_all2all.custom_kernel((cfg, mine, rank, world_size))  # CPU tensors, one node -> shared memory
        layer = host_ops.get_layer(cfg, rank, world_size)
        exact = oracle.moe_expected_output(cfg, mine, world_size)
        ok, msg = oracle.check_moe_output(y, exact)
        lay_ok, lay_msg = oracle.compare_dispatch_layout(
            (layer.expert_num_tokens, layer.expert_x, layer.expert_meta),
            oracle.moe_dispatch_oracle(cfg, [e[1] for e in everyone], rank),
        )
        res["ok"] &= bool(ok) and list(y.shape) == [mine.num_tokens, cfg.hidden_dim] and y.dtype == cfg.out_dtype
        res["msg"] = res["msg"] or msg
        res["layout_ok"] &= bool(lay_ok)
        res["layout_msg"] = res["layout_msg"] or lay_msg
        res["rel"] = max(res["rel"], oracle.relative_error(y, exact))
    res["cached_layers"] = len(host_ops._LAYERS)
    host_ops.release()
    return res


@pytest.mark.parametrize(
    "world_size,spec,rel",
    [
        (2, dict(E=16, k=2, H=256, T=32, seed=11, dtype="float32", fixed=32), 1e-6),
        (4, dict(E=8, k=2, H=64, T=4, seed=1236, dtype="float16", weights="rand"), 2e-3),  # random token counts
        (8, dict(E=64, k=6, H=512, T=48, seed=5, dtype="bfloat16", routing="zipf"), 1e-2),
    ],
)
def test_moe_over_shared_memory_matches_the_oracle_call_after_call(world_size, spec, rel):
    for r in run_ranks(_moe_rank, world_size, "gloo", (spec, 3), 300.0):
        assert r["ok"], r["msg"]
        assert r["layout_ok"], r["layout_msg"]  # reference row order: source rank, then (token, k)
        assert r["rel"] < rel
        assert r["cached_layers"] == 1


def _moe_dedup_rank(rank, world_size, spec, calls):
    _patient()
    from amd_distributed_2025_b200.models.host_ops import HostMoEAllToAll

    res = {"ok": True, "msg": "", "layout_ok": True, "layout_msg": "", "rel": 0.0}
    cfg = _moe_inputs(spec, spec["seed"], world_size)[rank][0]
    # every rank cuts its tokens into a different number of chunks: the owners learn it from the info word
    layer = HostMoEAllToAll(cfg, rank, world_size, mode="dedup", chunks=1 + (rank + spec.get("chunk_shift", 0)) % 4,
                            partial_dtype=torch.float32 if spec.get("fp32_partials") else None)
    for call in range(calls):
        everyone = _moe_inputs(spec, spec["seed"] + 17 * call, world_size)
        cfg, mine, _, _ = everyone[rank]
        n = mine.num_tokens
        num, ex, em = layer.dispatch(mine.x, mine.indices[:n])
        lay_ok, lay_msg = oracle.compare_dispatch_layout((num, ex, em), oracle.moe_dispatch_oracle(cfg, [e[1] for e in everyone], rank))
        if call % 2:
            # an expert output that does not live in the slab: the owner reduces it locally
            ey = (ex.to(cfg.out_dtype) * (1 + rank)).clone()
        else:
            ey = layer.expert_scale(1 + rank)
        y = torch.empty(n, cfg.hidden_dim, dtype=cfg.out_dtype)
        layer.combine(y, mine.weights[:n], ey)
        exact = oracle.moe_expected_output(cfg, mine, world_size)
        ok, msg = oracle.check_moe_output(y, exact)
        res["ok"] &= bool(ok)
        res["msg"] = res["msg"] or msg
        res["layout_ok"] &= bool(lay_ok)
        res["layout_msg"] = res["layout_msg"] or lay_msg
        res["rel"] = max(res["rel"], oracle.relative_error(y, exact))
    layer.close()
    return res


@pytest.mark.parametrize(
    "world_size,spec,rel",
    [
        (1, dict(E=8, k=2, H=64, T=16, seed=3, dtype="float32"), 1e-6),
        (2, dict(E=16, k=2, H=256, T=32, seed=11, dtype="float32", fixed=32), 1e-6),
        (3, dict(E=9, k=3, H=40, T=7, seed=29, dtype="float16", weights="rand", chunk_shift=2), 2e-3),
        (4, dict(E=8, k=2, H=64, T=4, seed=1236, dtype="float16", weights="rand"), 2e-3),  # random token counts, some zero
        (8, dict(E=64, k=6, H=512, T=48, seed=5, dtype="bfloat16", routing="zipf", fp32_partials=True), 1e-2),
        (8, dict(E=64, k=6, H=512, T=48, seed=6, dtype="bfloat16", routing="zipf", chunk_shift=1), 2e-2),
    ],
)
def test_moe_dedup_protocol_between_cpu_ranks(world_size, spec, rel):
    """The device kernels' default protocol (one row per destination rank, records, chunk flags
    announced through the info word, owner-side pre-reduction, one row back per owner) between
    real processes, call after call on the same buffers."""
    for r in run_ranks(_moe_dedup_rank, world_size, "gloo", (spec, 4), 300.0):
        assert r["ok"], r["msg"]
        assert r["layout_ok"], r["layout_msg"]
        assert r["rel"] < rel


def _modes_agree(rank, world_size):
    _patient()
    from amd_distributed_2025_b200.models import host_ops, moe_all2all

    cfg, mine, _, _ = contract.make_moe_inputs(16, 4, 128, 16, 3, rank, world_size, device=CPU, dtype=torch.float32,
                                               weights="softmax")
    data = (cfg, mine, rank, world_size)
    a = moe_all2all.custom_kernel(data, backend="shm", mode="direct")
    b = moe_all2all.custom_kernel(data, backend="shm", mode="dedup")
    host_ops.release()
    return {"max_diff": float((a - b).abs().max()) if a.numel() else 0.0}


def test_direct_and_dedup_protocols_agree_through_custom_kernel():
    for r in run_ranks(_modes_agree, 4, "gloo", (), 300.0):
        assert r["max_diff"] < 1e-5


def _some_ranks_without_tokens(rank, world_size):
    _patient()
    from amd_distributed_2025_b200.models.host_ops import HostMoEAllToAll

    cfg = contract.MoEConfig(num_experts=8, experts_per_token=2, hidden_dim=32, max_num_tokens=8, in_dtype=torch.float32,
                             out_dtype=torch.float32)
    worst = 0.0
    for mode in ("direct", "dedup"):
        layer = HostMoEAllToAll(cfg, rank, world_size, mode=mode, chunks=3)
        for call in range(4):
            gen = torch.Generator().manual_seed(100 * call + rank)
            tokens = 0 if (rank + call) % 2 == 0 else 5  # every other rank sends nothing, alternating per call
            x = torch.randn(tokens, 32, generator=gen)
            idx = (torch.stack([torch.randperm(8, generator=gen)[:2] for _ in range(tokens)]).to(torch.int32)
                   if tokens else torch.zeros(0, 2, dtype=torch.int32))
            w = torch.rand(tokens, 2, generator=gen)
            y = layer.forward(x, idx, w, 2.0)  # the same scale on every owner: y = 2 x sum_k w_k
            if tokens:
                worst = max(worst, float((y - 2.0 * x * w.sum(1, keepdim=True)).abs().max()))
            assert list(y.shape) == [tokens, 32]
        layer.close()
    return {"err": worst}


def test_ranks_without_tokens_still_take_part_in_every_exchange():
    for r in run_ranks(_some_ranks_without_tokens, 4, "gloo", (), 300.0):
        assert r["err"] < 1e-5


def _many_calls(rank, world_size, calls):
    _patient()
    from amd_distributed_2025_b200.models.host_ops import HostGemmRS, HostMoEAllToAll

    torch.set_num_threads(1)
    cfg = contract.MoEConfig(num_experts=8, experts_per_token=3, hidden_dim=24, max_num_tokens=6, in_dtype=torch.float32,
                             out_dtype=torch.float32)
    layers = [HostMoEAllToAll(cfg, rank, world_size, mode="direct"),
              HostMoEAllToAll(cfg, rank, world_size, mode="dedup", chunks=2)]
    op = HostGemmRS(world_size * 8 * 16 * 4, rank, world_size)
    worst = 0.0
    for call in range(calls):
        gen = torch.Generator().manual_seed(7919 * call + rank)
        tokens = int(torch.randint(0, 7, (1,), generator=gen))
        x = torch.randn(tokens, 24, generator=gen)
        idx = (torch.stack([torch.randperm(8, generator=gen)[:3] for _ in range(tokens)]).to(torch.int32)
               if tokens else torch.zeros(0, 3, dtype=torch.int32))
        w = torch.rand(tokens, 3, generator=gen)
        y = layers[call % 2].forward(x, idx, w, 1.5)
        if tokens:
            worst = max(worst, float((y - 1.5 * x * w.sum(1, keepdim=True)).abs().max()))
        # a reduce-scatter in between, its shape changing from call to call (same two parities)
        m = world_size * (1 + call % 8)
        a = torch.full((m, 4), float(rank + 1))
        wt = torch.ones(16, 4)
        out = op(a, wt)
        want = 4.0 * sum(range(1, world_size + 1))
        worst = max(worst, float((out - want).abs().max()))
    for layer in layers:
        layer.close()
    op.close()
    return {"err": worst}


def test_hundreds_of_back_to_back_calls_with_changing_sizes_need_no_barrier():
    """Flag epochs, chunk flag values and the two staging parities over 300 calls whose token counts
    (zero included) and row counts change every call, three operators interleaved on every rank."""
    for r in run_ranks(_many_calls, 4, "gloo", (300,), 600.0):
        assert r["err"] < 1e-4


def _gemm_rank(rank, world_size, m, n, k, calls):
    _patient()
    from amd_distributed_2025_b200.models import gemm_rs, host_ops

    res = {"ok": True, "msg": "", "rel": 0.0, "once_ok": True}
    for call in range(calls):
        everyone = [contract.make_gemm_rs_inputs(r, world_size, m, n, k, True, 5 + call, device=CPU) for r in range(world_size)]
        a_all, w_all, bias = [e[0] for e in everyone], [e[1] for e in everyone], everyone[rank][2]
        out = gemm_rs.custom_kernel(everyone[rank])  # bias on every rank, as the reference does
        ok, msg = oracle.check_gemm_rs_output(out, oracle.gemm_rs_fused_rounding(a_all, w_all, bias, rank))
        res["ok"] &= bool(ok) and list(out.shape) == [m // world_size, n]
        res["msg"] = res["msg"] or msg
        res["rel"] = max(res["rel"], oracle.relative_error(out, oracle.gemm_rs_truth(a_all, w_all, bias, rank)))
        once = gemm_rs.custom_kernel(everyone[rank], bias_mode="once")
        no_bias = oracle.gemm_rs_truth(a_all, w_all, None, rank)
        res["once_ok"] &= oracle.relative_error(once, no_bias + bias.to(no_bias.dtype)) < 1e-2
    host_ops.release()
    return res


@pytest.mark.parametrize("world_size,m,n,k", [(2, 64, 48, 256), (4, 128, 96, 512), (8, 64, 40, 1024)])
def test_gemm_rs_over_shared_memory_alternates_parities_without_barriers(world_size, m, n, k):
    # 3 calls x 2 bias modes = 6 operator calls in a row on the same two staging parities
    for r in run_ranks(_gemm_rank, world_size, "gloo", (m, n, k, 3), 300.0):
        assert r["ok"], r["msg"]
        assert r["rel"] < 1e-2
        assert r["once_ok"]


def _backends_agree(rank, world_size):
    _patient()
    from amd_distributed_2025_b200.models import moe_all2all

    cfg, mine, _, _ = contract.make_moe_inputs(16, 4, 128, 16, 3, rank, world_size, device=CPU, dtype=torch.float32,
                                               fixed_num_tokens=16, weights="softmax")
    data = (cfg, mine, rank, world_size)
    a = moe_all2all.custom_kernel(data, backend="shm")
    b = moe_all2all.custom_kernel(data, backend="torch")
    return {"max_diff": float((a - b).abs().max())}


def test_shared_memory_and_library_collective_backends_agree():
    for r in run_ranks(_backends_agree, 2, "gloo", (), 300.0):
        assert r["max_diff"] < 1e-5


# -- failure detection: a rank that stops calling ------------------------------------------

def _leaver(prefix, rank, world_size, q, mode):
    from amd_distributed_2025_b200.contract import MoEConfig
    from amd_distributed_2025_b200.models.host_ops import HostMoEAllToAll
    from amd_distributed_2025_b200.utils.status import StatusError

    torch.set_num_threads(1)
    cfg = MoEConfig(num_experts=9, experts_per_token=2, hidden_dim=32, max_num_tokens=8, in_dtype=torch.float32,
                    out_dtype=torch.float32)
    layer = HostMoEAllToAll(cfg, rank, world_size, prefix=prefix, wait_limit_ms=300.0, mode=mode)
    gen = torch.Generator().manual_seed(rank)
    x = torch.randn(8, 32, generator=gen)
    idx = torch.stack([torch.randperm(9, generator=gen)[:2] for _ in range(8)]).to(torch.int32)
    w = torch.full((8, 2), 0.5)
    layer.forward(x, idx, w, 1.0)  # step 1: everybody takes part
    if rank == world_size - 1:
        q.put((rank, "left", None, None, 0.0))  # leaves between steps, nothing in flight
        return
    t0 = time.perf_counter()
    try:
        layer.forward(x, idx, w, 1.0)
        q.put((rank, "no error", None, None, time.perf_counter() - t0))
    except StatusError as exc:
        q.put((rank, exc.code, exc.phase, exc.status["peer"], time.perf_counter() - t0))


@pytest.mark.parametrize("mode", ["direct", "dedup"])
def test_a_rank_that_leaves_between_steps_ends_the_others_wait_with_a_status(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    prefix = f"b200_test_leave_{mode}_{os.getpid()}"
    procs = [ctx.Process(target=_leaver, args=(prefix, r, 3, q, mode)) for r in range(3)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert got[2][1] == "left"
    for rank, code, phase, peer, seconds in got[:2]:
        assert (code, phase, peer) == ("timeout", "moe_counts", 2)
        assert 0.25 < seconds < 10.0  # gave up after the limit, not much later


def test_single_process_world_of_one_needs_no_process_group():
    from amd_distributed_2025_b200.models import gemm_rs, host_ops, moe_all2all

    cfg, d, _, _ = contract.make_moe_inputs(8, 2, 64, 16, 1, 0, 1, device=CPU, dtype=torch.float32)
    y = moe_all2all.custom_kernel((cfg, d, 0, 1))
    ok, msg = oracle.check_moe_output(y, oracle.moe_expected_output(cfg, d, 1))
    assert ok, msg
    a, w, b = contract.make_gemm_rs_inputs(0, 1, 32, 48, 64, True, 3, device=CPU)
    out = gemm_rs.custom_kernel((a, w, b))
    ok, msg = oracle.check_gemm_rs_output(out, oracle.gemm_rs_fused_rounding([a], [w], b, 0))
    assert ok, msg
    host_ops.release()


def _dispatch_twice(rank, world_size, mode):
    _patient()
    import time as _time

    from amd_distributed_2025_b200.models.host_ops import HostMoEAllToAll

    cfg = contract.MoEConfig(num_experts=4, experts_per_token=2, hidden_dim=16, max_num_tokens=4, in_dtype=torch.float32,
                             out_dtype=torch.float32)
    layer = HostMoEAllToAll(cfg, rank, world_size, mode=mode)
    idx = torch.tensor([[0, 2], [1, 3], [2, 0], [3, 1]], dtype=torch.int32)
    first = torch.full((4, 16), 1.0 + rank)
    second = torch.full((4, 16), 100.0 + rank)
    num, ex, _ = layer.dispatch(first, idx)
    if rank == 0:
        _time.sleep(0.5)  # this rank's caller is slow to look at what it received ...
    seen = ex.clone()     # ... and must still find the FIRST dispatch's rows, whatever the others do meanwhile
    layer.dispatch(second, idx)
    after = layer.expert_x.clone()
    layer.close()
    return {"first_ok": bool((seen[:, :4] < 50.0).all()), "second_ok": bool((after[:, :4] > 50.0).all()),
            "rows": int(num.sum())}


@pytest.mark.parametrize("mode", ["direct", "dedup"])
def test_a_second_dispatch_never_overwrites_rows_a_slow_rank_still_reads(mode):
    for r in run_ranks(_dispatch_twice, 2, "gloo", (mode,), 300.0):
        assert r["rows"] == 8  # 4 tokens x 2 entries x 2 ranks over 4 experts: 4 rows per expert, 2 experts per rank
        assert r["first_ok"] and r["second_ok"]
