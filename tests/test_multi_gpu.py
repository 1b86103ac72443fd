"""Multi-GPU tests: the fused kernels on 2..8 ranks (one process per GPU, NCCL only for
bootstrap) against the communication-free oracles."""
import pytest
import torch

from amd_distributed_2025_b200 import contract, oracle
from amd_distributed_2025_b200.harness.eval import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _world_sizes():
    """2, 4 and 8 ranks as far as the box has GPUs; ``B200_TEST_WORLD_SIZES=4,8`` narrows the list
    (a large box need not repeat what a small one has already run)."""
    import os

    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    want = [int(w) for w in os.environ.get("B200_TEST_WORLD_SIZES", "2,4,8").split(",") if w.strip()]
    return [w for w in want if w <= n] or [2]


MOE_SHAPES = [
    # (num_experts, k, hidden, max_num_tokens, seed, fixed tokens per rank or None, routing)
    # -- from the task's test list (random token count per rank, as the reference generates it)
    (8, 2, 6144, 4, 1236, None, "uniform"),
    (64, 6, 2048, 8, 542, None, "uniform"),
    (128, 4, 2880, 32, 51, None, "uniform"),
    (128, 8, 4096, 128, 534, None, "uniform"),
    (256, 8, 7168, 64, 897, None, "uniform"),
    # -- more than 4096 (token, k) entries per rank: the grid-barrier dispatch kernels
    (64, 6, 512, 1024, 77, 1024, "zipf"),
    (64, 6, 512, 1024, 78, 1000, "uniform"),
    (16, 8, 1024, 768, 79, 768, "zipf"),
]


def _moe_inputs(shape, it, world_size, dev):
    """Inputs of every rank for iteration ``it``: a new seed each time and, for the fixed-size
    shapes, a different token count, so that a row or flag left over from the previous call
    cannot pass for the current one."""
    E, k, H, T, seed, fixed, routing = shape
    seed = seed + 7919 * it
    if fixed is None:
        return [contract.generate_moe_input(E, k, H, T, seed, r, world_size, device=dev) for r in range(world_size)]
    n_tok = max(fixed - 37 * it, 1)
    return [contract.make_moe_inputs(E, k, H, T, seed, r, world_size, device=dev, dtype=torch.bfloat16,
                                     fixed_num_tokens=n_tok, routing=routing, weights="softmax")
            for r in range(world_size)]


def _moe_rank(rank, world_size, shapes, repeats, modes, env=None):
    import os

    from amd_distributed_2025_b200.models import moe_all2all

    os.environ.update(env or {})  # knobs that a layer reads when it is created

    dev = torch.device("cuda", torch.cuda.current_device())
    out = []
    for mode in modes:
        for shape in shapes:
            E, k, H, T = shape[:4]
            if E % world_size:
                continue
            res = {"shape": [mode] + list(shape[:4]), "ok": True, "msg": "", "layout_ok": True, "layout_msg": ""}
            for it in range(repeats):
                everyone = _moe_inputs(shape, it, world_size, dev)
                cfg, mine, _, _ = everyone[rank]
                layer = moe_all2all.get_layer(cfg, rank, world_size, mode=mode)
                if it % 2 == 0:
                    # the three-call API: dispatch, the expert op as its own kernel, combine
                    got = layer.dispatch(mine.x, mine.indices)
                    torch.cuda.synchronize()
                    lay_ok, lay_msg = oracle.compare_dispatch_layout(
                        got, oracle.moe_dispatch_oracle(cfg, [e[1] for e in everyone], rank))
                    if not lay_ok:
                        res["layout_ok"], res["layout_msg"] = False, f"iteration {it}: {lay_msg}"
                    layer.expert_scale(1 + rank)
                    y = torch.empty(mine.num_tokens, H, dtype=cfg.out_dtype, device=dev)
                    layer.combine(y, mine.weights, got[2], layer.expert_y, got[0], mine.num_tokens)
                else:
                    y = moe_all2all.custom_kernel((cfg, mine, rank, world_size), mode=mode)
                torch.cuda.synchronize()
                try:
                    layer.check()
                except Exception as exc:  # noqa: BLE001
                    res["ok"], res["msg"] = False, f"iteration {it}: {exc}"
                    break
                # fp16 (the task's type): against the reference's own rounding points; bf16: against the
                # exact sum, because eight bf16 roundings of the accumulator alone stray further from
                # it than the task tolerance
                want = oracle.moe_expected_output(cfg, mine, world_size,
                                                  emulate_reference_rounding=cfg.out_dtype == torch.float16)
                ok2, msg2 = oracle.check_moe_output(y, want)
                rel = oracle.relative_error(y, oracle.moe_expected_output(cfg, mine, world_size, acc_dtype=torch.float64))
                if not ok2 or rel > 5e-3:
                    res["ok"], res["msg"] = False, f"iteration {it}: {msg2} rel {rel:.3e}"
            out.append(res)
    torch.cuda.synchronize()
    moe_all2all.release_layers()
    return out


@pytest.mark.parametrize("ws", _world_sizes())
def test_moe_dispatch_combine_multi_rank(ws):
    for per_rank in run_ranks(_moe_rank, ws, "nccl", (MOE_SHAPES, 4, ("dedup", "direct")), 900.0):
        assert per_rank, "no shape ran"
        for r in per_rank:
            assert r["layout_ok"], (r["shape"], r["layout_msg"])
            assert r["ok"], (r["shape"], r["msg"])


@pytest.mark.parametrize("ws", _world_sizes())
def test_moe_chunked_dispatch_multi_rank(ws):
    """The chunked form of the large dispatch (several "delivered" flags per source, replication
    of chunk c while c + 1 is in flight), forced on for shapes and world sizes below its
    thresholds, with 3 and with 4 chunks."""
    big = [s for s in MOE_SHAPES if s[5] is not None]
    for chunks in ("3", "4"):
        env = {"B200_MOE_CHUNK_MIN_RANKS": "2", "B200_MOE_CHUNK_MIN_BYTES": "0", "B200_MOE_CHUNKS": chunks}
        for per_rank in run_ranks(_moe_rank, ws, "nccl", (big, 3, ("dedup",), env), 900.0):
            assert per_rank, "no shape ran"
            for r in per_rank:
                assert r["layout_ok"], (chunks, r["shape"], r["layout_msg"])
                assert r["ok"], (chunks, r["shape"], r["msg"])


GEMM_SHAPES = [
    # (m, n, k, has_bias, seed, operand distribution) -- task test shapes plus small/ragged ones
    (64, 2880, 2880, True, 2035, "reference"),
    (512, 3584, 14336, True, 4297, "reference"),
    (2048, 4096, 7168, False, 716, "reference"),
    (64, 2880, 2880, True, 2035, "normal"),
    (512, 3584, 14336, True, 4297, "normal"),
    (4096, 2880, 2880, True, 136, "normal"),
    (256, 5120, 12800, True, 61, "normal"),
    (8192, 8192, 28672, False, 1536, "normal"),
]


def _gemm_check(rank, world_size, spec, seed, y, everyone):
    m, n, k, has_bias, _, kind = spec
    from amd_distributed_2025_b200.parallel.baseline_nccl import gemm_rs_torch

    data = everyone[rank]
    a_all, w_all = [e[0] for e in everyone], [e[1] for e in everyone]
    truth = oracle.gemm_rs_truth(a_all, w_all, data[2], rank, dtype=torch.float32)
    rel = oracle.relative_error(y, truth)
    lib = gemm_rs_torch(data)  # library GEMM + NCCL reduce-scatter: what the task's checker computes
    if kind == "reference":
        ok2, msg2 = oracle.check_gemm_rs_output(y, lib)
        outliers = 0.0
    else:
        # Same rounding chain (bf16 partials, fp32 sum): all but a handful of elements must agree
        # within the task tolerance.  The library path also rounds after every hop of its ring;
        # with unit-variance operands that alone moves about 1 % of its elements further than the
        # tolerance from the same-chain result (see oracle.outlier_fraction), so it is only a
        # loose sanity bound here.
        want = oracle.gemm_rs_fused_rounding(a_all, w_all, data[2], rank)
        outliers = oracle.outlier_fraction(y, want, oracle.GEMM_RS_RTOL, oracle.GEMM_RS_ATOL)
        vs_lib = oracle.outlier_fraction(y, lib, oracle.GEMM_RS_RTOL, oracle.GEMM_RS_ATOL)
        ok2 = outliers < 1e-3 and vs_lib < 3e-2
        msg2 = f"{outliers:.2e} (same chain) / {vs_lib:.2e} (library) of the elements outside the task tolerance"
    return bool(ok2 and rel < 5e-3), msg2, rel, outliers


def _gemm_rank(rank, world_size, shapes, repeats, rs_mode="p2p"):
    import os

    from amd_distributed_2025_b200.models import gemm_rs

    os.environ["B200_RS_MODE"] = rs_mode  # read when the cached operator creates its workspace
    dev = torch.device("cuda", torch.cuda.current_device())
    out = []
    usable = [s for s in shapes if not (s[0] % world_size or s[2] % world_size or (s[2] // world_size) % 8)]
    for i, spec in enumerate(usable):
        m, n, k, has_bias, seed, kind = spec
        # a second, smaller shape alternates with the one under test on the same cached operator:
        # consecutive calls use the other staging parity and different tile counts, with no
        # barrier in between; every call gets new operands and every result is checked
        other = usable[(i + 1) % len(usable)] if m * n <= 4096 * 4096 else None
        res = {"shape": [m, n, k, kind], "ok": True, "msg": "", "rel": 0.0, "outliers": 0.0}
        big = m * n * k > 2 ** 36
        for it in range(1 if big else repeats):
            calls = [(spec, seed + 101 * it)]
            if other is not None and other[0] * other[1] <= 4096 * 4096:
                calls.append((other, other[4] + 101 * it + 1))
            pending = []
            for sp, sd in calls:
                everyone = [contract.make_gemm_rs_inputs(r, world_size, sp[0], sp[1], sp[2], sp[3], sd, device=dev, dist=sp[5])
                            for r in range(world_size)]
                pending.append((sp, sd, gemm_rs.custom_kernel(everyone[rank]), everyone))
            if big:  # the largest shape once more on the other parity, same operands
                pending.append((spec, seed, gemm_rs.custom_kernel(pending[0][3][rank]), pending[0][3]))
            torch.cuda.synchronize()
            try:
                op = gemm_rs.get_op(m, n, k // world_size)
                res["rs_mode"], res["rs_mode_note"] = op.rs_mode, op.rs_mode_note
                op.check()
            except Exception as exc:  # noqa: BLE001
                res["ok"], res["msg"] = False, str(exc)
                break
            for sp, sd, y, everyone in pending:
                ok, msg, rel, outl = _gemm_check(rank, world_size, sp, sd, y, everyone)
                res["rel"], res["outliers"] = max(res["rel"], rel), max(res["outliers"], outl)
                if not ok:
                    res["ok"], res["msg"] = False, f"iteration {it}, {list(sp[:3])}: {msg}"
            del pending
        out.append(res)
    torch.cuda.synchronize()
    gemm_rs.release_ops()
    return out


@pytest.mark.parametrize("rs_mode", ["p2p", "nvls"])
@pytest.mark.parametrize("ws", _world_sizes())
def test_gemm_rs_multi_rank(ws, rs_mode):
    """"p2p": partial tiles are stored into the owners' memory; "nvls": they stay with their
    producer and the owner pulls their sum through NVSwitch.  Same results either way."""
    results = run_ranks(_gemm_rank, ws, "nccl", (GEMM_SHAPES, 3, rs_mode), 900.0)
    for per_rank in results:
        assert per_rank, "no shape ran"
        for r in per_rank:
            assert r["ok"], (r["shape"], r["msg"], r["rel"], r["outliers"])
    ran = {r.get("rs_mode") for per_rank in results for r in per_rank}
    if rs_mode == "nvls" and ran != {"nvls"}:
        pytest.skip("NVLink multicast unavailable, the peer-to-peer path ran instead: " + results[0][0].get("rs_mode_note", ""))


def _mcast_rank(rank, world_size):
    """Multicast region: every rank fills its part with (rank + 1), the in-switch sum must be
    1 + 2 + ... + world_size everywhere.  Reports "unavailable" where the box offers no NVLS."""
    from amd_distributed_2025_b200.parallel.symm_mem import McastWorkspace

    ok, why = McastWorkspace.probe()
    if not ok:
        return {"available": False, "why": why}
    try:
        ws = McastWorkspace(4 << 20, rank=rank, world_size=world_size)
    except RuntimeError as exc:
        return {"available": False, "why": str(exc)}
    try:
        n = 1 << 16
        ws.view(0, (n,), torch.bfloat16).fill_(float(rank + 1))
        torch.cuda.synchronize()
        torch.distributed.barrier()
        out = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
        ws.region.reduce_selftest(0, out)
        torch.cuda.synchronize()
        want = float(world_size * (world_size + 1) // 2)
        good = bool((out.float() == want).all())
        torch.distributed.barrier()
    finally:
        # whatever happened above: no rank leaves while its memory is bound to the multicast object
        ws.close(collective=True)
    return {"available": True, "ok": good, "got": float(out[0]), "want": want}


@pytest.mark.parametrize("ws", _world_sizes())
def test_multicast_region_sums_in_the_switch(ws):
    res = run_ranks(_mcast_rank, ws, "nccl", (), 300.0)
    if not all(r["available"] for r in res):
        pytest.skip("NVLink multicast unavailable: " + "; ".join(sorted({r.get("why", "") for r in res if not r["available"]})))
    for r in res:
        assert r["ok"], r
