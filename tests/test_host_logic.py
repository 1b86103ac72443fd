"""CPU tests of the host-side logic: slab layouts, epochs, the GEMM planner, status decoding,
timing and roofline helpers.  The native extension is built if it is missing (nvcc
cross-compiles without a GPU); nothing here launches a kernel."""
import math

import pytest
import torch

from amd_distributed_2025_b200 import contract
from amd_distributed_2025_b200.parallel.symm_mem import EpochCounter, SlabLayout
from amd_distributed_2025_b200.utils import roofline, timing
from amd_distributed_2025_b200.utils.status import StatusError, describe_status


@pytest.fixture(scope="module")
def ext():
    from amd_distributed_2025_b200.ops import _ext

    return _ext.load()


def test_slab_layout_is_deterministic_aligned_and_disjoint():
    a, b = SlabLayout(4096), SlabLayout(4096)
    for lay in (a, b):
        lay.add("counts", 8 * 256 * 4)
        lay.add("meta", 32 * 2048 * 5 * 4)
        lay.add("x", 32 * 2048 * 7168 * 2)
    assert a.regions == b.regions  # every rank derives the same offsets without talking
    assert not a.overlaps()
    assert all(off % 1024 == 0 and off >= 4096 for off, _ in a.regions.values())
    assert a.total_bytes >= max(off + size for off, size in a.regions.values())
    with pytest.raises(KeyError):
        a.add("x", 16)


def test_moe_slab_layout_sizes_match_the_dispatch_contract():
    from amd_distributed_2025_b200.models.moe_all2all import moe_slab_layout

    cfg = contract.MoEConfig(256, 8, 7168, 256, torch.bfloat16, torch.bfloat16)
    lay = moe_slab_layout(cfg, 8, 4096)
    rows = 32 * 2048  # E_local * max_recv
    assert lay.size("expert_x") == rows * 7168 * 2 and lay.size("expert_y") == rows * 7168 * 2
    assert lay.size("expert_meta") == rows * 5 * 4 and lay.size("counts") == 8 * 256 * 4
    assert not lay.overlaps()


def test_epochs_only_grow_per_protocol():
    e = EpochCounter()
    assert [e.next("a"), e.next("a"), e.next("b"), e.next("a")] == [1, 2, 1, 3]
    assert e.current("a") == 3 and e.current("missing") == 0


def test_status_decoding():
    st = {"code": 1, "phase": 5, "peer": 3, "detail": 17, "epoch": 9, "seen": 2}
    text = describe_status(st, rank=4)
    assert "timeout" in text and "rs_partials" in text and "rank 4" in text
    err = StatusError(text, st)
    assert err.code == "timeout" and err.phase == "rs_partials" and err.status["peer"] == 3


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
def test_gemm_plan_is_valid_for_all_task_shapes(ext, ws):
    specs = contract.task_specs("gemm_rs", "tests") + contract.task_specs("gemm_rs", "benchmarks")
    specs += [dict(m=c["m"], n=c["n"], k=c["k"]) for c in contract.load_task("headline")["gemm_rs"]]
    for s in specs:
        if s["m"] % ws or s["k"] % ws:
            continue
        m, n, k = s["m"], s["n"], s["k"] // ws
        plan = ext.gemm_rs_plan(m, n, k, ws, 0, -1, 0)
        assert plan == ext.gemm_rs_plan(m, n, k, ws, 0, -1, 0)  # pure function: all ranks agree
        assert plan["block_n"] in (64, 128, 192, 256) and plan["cta_pair"] in (0, 1)
        if plan["cta_pair"]:
            assert plan["block_n"] != 64
        num_kb = (k + 63) // 64
        sp = plan["splits"]
        assert 1 <= sp <= 8 and (sp - 1) * math.ceil(num_kb / sp) < num_kb  # no empty K slice
        assert plan["stage_bytes"] == (m * n * 2 if sp == 1 else sp * m * n * 4)
        assert plan["counter_bytes"] >= math.ceil(m / 128) * math.ceil(n / 64) * 4 * 4


def test_gemm_plan_honours_overrides_and_prefers_pairs_for_large_problems(ext):
    assert ext.gemm_rs_plan(8192, 8192, 3584, 8, 0, -1, 0)["cta_pair"] == 1
    assert ext.gemm_rs_plan(8192, 8192, 3584, 8, 0, -1, 0)["splits"] == 1
    forced = ext.gemm_rs_plan(2048, 2048, 2048, 1, 128, 0, 2)
    assert (forced["block_n"], forced["cta_pair"], forced["splits"]) == (128, 0, 2)
    # a problem that leaves most SMs idle gets its K cut on one GPU
    assert ext.gemm_rs_plan(256, 5120, 12800, 1, 0, -1, 0)["splits"] > 1


def test_noalloc_entry_point_is_exported(ext):
    import ctypes

    lib = ctypes.CDLL(ext.__file__)
    assert hasattr(lib, "b200_moe_dispatch_noalloc") and hasattr(lib, "b200_moe_dispatch_noalloc_status")


def test_geomean_and_summaries():
    assert timing.geomean([1.0, 100.0]) == pytest.approx(10.0)
    assert math.isnan(timing.geomean([]))
    s = timing.summarize([3.0, 1.0, 2.0])
    assert s["min_ms"] == 1.0 and s["median_ms"] == 2.0 and s["n"] == 3


def test_roofline_arithmetic():
    peaks = {"bf16_tflops": 1600.0, "bf16_tflops_sustained": 1400.0, "nvlink_gbs_per_dir": 770.0}
    r = roofline.gemm_rs_roofline_us(8192, 8192, 28672, 8, peaks)
    assert r["flops"] == pytest.approx(2 * 8192 * 8192 * 3584)
    assert r["compute_us"] == pytest.approx(r["flops"] / 1400e12 * 1e6)
    assert r["link_bytes"] == pytest.approx(7 / 8 * 8192 * 8192 * 2)
    assert r["roofline_us"] == max(r["compute_us"], r["link_us"])
    m = roofline.moe_roofline_us(896, 896, 14336, peaks)
    assert m["roofline_us"] == pytest.approx(2 * 896 * 14336 / 770e9 * 1e6)
    loaded = roofline.load_peaks()
    assert loaded["source"] in ("measured", "fallback") and loaded["hbm_gbs"] > 1000


def test_roofline_report_for_a_bench_line():
    line = {"n_gpus": 8, "per_config_us": {
        "moe_decode": {"us": 140.0}, "gemm_rs_large": {"us": 480.0}, "gemm_rs_sweep_m256": {"us": 100.0}}}
    peaks = {"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1400.0, "nvlink_gbs_per_dir": 770.0}
    rep = roofline.report(line, peaks)
    assert set(rep) == set(line["per_config_us"])
    big = rep["gemm_rs_large"]
    assert big["roofline_us"] == pytest.approx(2 * 8192 * 8192 * 3584 / 1400e12 * 1e6)
    assert big["fraction_of_roofline"] == pytest.approx(big["roofline_us"] / 480.0)
    # decode: a token reaches 8 * (1 - (7/8)^8) = 5.25 distinct ranks, 7/8 of them remote: about
    # 128 * 5.25 * 7/8 = 590 rows of 14 336 bytes leave every rank, once per phase
    assert 18.0 < rep["moe_decode"]["roofline_us"] < 28.0


def test_report_table_has_ratios_geomeans_and_the_speed_of_light_column():
    from amd_distributed_2025_b200.harness import report

    specs = contract.task_specs("gemm_rs", "benchmarks")[:2]
    by_arm = {
        "ours": [{"spec": specs[0], "ok": True, "time_us": 50.0}, {"spec": specs[1], "ok": True, "time_us": 200.0}],
        "torch": [{"spec": specs[0], "ok": True, "time_us": 100.0}, {"spec": specs[1], "ok": False, "time_us": 800.0}],
    }
    text = report.render("gemm_rs", 8, by_arm)
    rows = [r for r in text.splitlines() if r.startswith("|")]
    assert len(rows) == 2 + 2 + 1  # header, rule, two shapes, geometric mean
    assert "2.00x" in rows[2] and "4.00x" in rows[3]
    assert "FAILS: torch" in rows[3] and "passes" in rows[2]
    assert "**100.0**" in rows[4] and "**282.8**" in rows[4] and "2.83x" in rows[4]
    sol = report.speed_of_light("gemm_rs")
    assert len(sol) >= 6 and all(v > 0 for v in sol.values())
    assert f"{sol[report._shape_key('gemm_rs', specs[0])]:.2f}" in rows[2]


def test_clock_sampler_only_reads_and_summarises_the_samples_under_load(monkeypatch):
    """Against a fake NVML: the sampler calls getters only, takes the median SM clock of the
    samples under load and decodes the throttle reasons seen there."""
    import sys
    import time
    import types

    from amd_distributed_2025_b200.utils.clocks import ClockSampler

    calls = []
    script = [(1965, 200_000, 0x0), (1305, 990_000, 0x4), (1290, 1_000_000, 0x4), (1320, 980_000, 0x4 | 0x20)]
    state = {"i": 0}

    class FakeNvml(types.ModuleType):
        NVML_CLOCK_SM = 1

        def __getattr__(self, name):  # anything that is not one of the getters below: refuse
            raise AssertionError(f"the sampler touched {name}")

    fake = FakeNvml("pynvml")
    fake.nvmlInit = lambda: calls.append("init")
    fake.nvmlShutdown = lambda: calls.append("shutdown")
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965

    def cur():
        return script[min(state["i"], len(script) - 1)]

    fake.nvmlDeviceGetClockInfo = lambda h, kind: cur()[0]
    fake.nvmlDeviceGetPowerUsage = lambda h: cur()[1]

    def reasons(h):
        mask = cur()[2]
        state["i"] += 1
        return mask

    fake.nvmlDeviceGetCurrentClocksEventReasons = reasons
    monkeypatch.setitem(sys.modules, "pynvml", fake)

    s = ClockSampler(0, interval_s=0.001)
    s.start()
    deadline = time.time() + 5.0
    while state["i"] < len(script) + 2 and time.time() < deadline:
        time.sleep(0.002)
    out = s.stop()
    assert calls[0] == "init" and calls[-1] == "shutdown"
    assert out["sm_max_mhz"] == 1965
    assert 1290 <= out["sm_mhz"] <= 1320  # the idle 1965 MHz sample is not "under load"
    assert out["power_w_max"] == 1000.0
    assert out["reasons"] == ["sw_power_cap", "sw_thermal_slowdown"]
    assert out["samples_under_load"] < out["samples"]


def test_clock_sampler_resolves_the_device_by_uuid_under_a_device_mask(monkeypatch):
    """CUDA ordinal 0 of a masked process is physical GPU 5: the sampler must read GPU 5's
    clocks (handle by UUID), not those of physical GPU 0, which may be another user's."""
    import sys
    import types

    from amd_distributed_2025_b200.utils.clocks import ClockSampler

    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlInit = lambda: None
    fake.nvmlShutdown = lambda: None
    physical = {f"GPU-0000-{i}": ("handle", i) for i in range(8)}
    fake.nvmlDeviceGetHandleByUUID = lambda u: physical[u if isinstance(u, str) else u.decode()]
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965
    fake.nvmlDeviceGetClockInfo = lambda h, kind: 1000 + h[1]  # a clock that tells which GPU was read
    fake.nvmlDeviceGetPowerUsage = lambda h: 500_000
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0
    monkeypatch.setitem(sys.modules, "pynvml", fake)

    s = ClockSampler(0, interval_s=0.001, uuid="0000-5")  # torch prints the UUID without the "GPU-" prefix
    s.start()
    out = s.stop()
    assert out["sm_mhz"] == 1005
    s = ClockSampler(3, interval_s=0.001)  # no UUID given: the index is all there is
    s.start()
    assert s.stop()["sm_mhz"] == 1003


def test_workspace_stays_poisoned_after_a_timeout_until_collective_recovery():
    """Arrival counters that are plain counts cannot be trusted after an expired wait (late
    arrivals of the failed call would satisfy the next one): a workspace created with
    ``poison_on_timeout`` keeps raising after ``reset_status`` until ``recover`` has zeroed the
    counters.  Driven here with a stand-in heap, no GPU."""
    from amd_distributed_2025_b200.parallel.symm_mem import SlabLayout, SymmetricWorkspace
    from amd_distributed_2025_b200.utils.status import StatusError

    class FakeHeap:
        def __init__(self):
            self.word = {"code": 0, "phase": 0, "peer": -1, "detail": 0, "epoch": 0, "seen": 0}
            self.mem = torch.full((8192,), 7, dtype=torch.uint8)

        def status_code(self):
            return self.word["code"]

        def status(self):
            return dict(self.word)

        status_sync = status

        def reset_status(self):
            self.word = dict(self.word, code=0)

        def view(self, off, shape, dtype):
            return self.mem[off:off + shape[0]]

    lay = SlabLayout(4096)
    lay.add("counters0", 256)
    lay.add("counters1", 256)
    for poison in (True, False):
        heap = FakeHeap()
        ws = SymmetricWorkspace(lay, rank=0, world_size=2, heap=heap, poison_on_timeout=poison)
        ws.check()
        ws.next_epoch("gemm_rs")
        heap.word.update(code=1, phase=5, peer=1)  # a peer's partial rows never arrived
        with pytest.raises(StatusError):
            ws.check()
        ws.reset_status()
        if not poison:
            ws.check()  # flags that carry the call number need no more than that
            continue
        with pytest.raises(StatusError) as err:
            ws.check()
        assert "recover" in str(err.value)
        ws.recover(("counters0", "counters1"))
        ws.check()
        assert int(heap.mem[4096:4096 + 256].sum()) == 0 and int(heap.mem[5120:5120 + 256].sum()) == 0
        assert ws.epochs.current("gemm_rs") == 0  # call numbers (and with them the staging parity) restart


def test_checked_layout_puts_a_guard_area_behind_every_region():
    from amd_distributed_2025_b200.parallel.symm_mem import SlabLayout

    plain, guarded = SlabLayout(4096), SlabLayout(4096, guard_bytes=1024)
    for lay in (plain, guarded):
        lay.add("a", 1000)
        lay.add("b", 5000)
    assert not plain.guards and len(guarded.guards) == 2
    (g0, n0), (g1, n1) = guarded.guards
    a_off, a_len = guarded.regions["a"]
    b_off, b_len = guarded.regions["b"]
    assert a_off + a_len <= g0 < g0 + n0 <= b_off and b_off + b_len <= g1 and g1 + n1 <= guarded.total_bytes
    assert not guarded.overlaps()


def test_gemm_rs_reserve_sizes_the_cached_workspace_once(monkeypatch):
    """``reserve`` with the task's shapes must leave a workspace that every later ``get_op`` of those
    shapes reuses (no free-and-recreate inside a serving loop); the env floor raises the first size."""
    from amd_distributed_2025_b200.models import gemm_rs as g

    built = []

    class FakeOp:
        def __init__(self, stage_bytes, counter_bytes, group=None):
            self.stage_bytes, self.counter_bytes, self._fits = stage_bytes, counter_bytes, set()
            built.append((stage_bytes, counter_bytes))

        def close(self, collective=False):
            pass

    monkeypatch.setattr(g, "GemmRS", FakeOp)
    monkeypatch.setattr(g, "_OPS", {})
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    monkeypatch.delenv("B200_RS_WORKSPACE_MB", raising=False)
    shapes = [(256, 5120, 12800), (8192, 8192, 28672), (2048, 5120, 12800), (64, 7168, 18432)]
    op = g.reserve(shapes)
    n_built = len(built)
    assert n_built <= 2 and op.stage_bytes >= 8192 * 8192 * 2
    for m, n, k in shapes:
        assert g.get_op(m, n, k) is op
    assert len(built) == n_built
    with pytest.raises(ValueError):
        g.reserve([])


def test_second_dedup_dispatch_without_combine_waits_for_all_ranks(monkeypatch):
    """Dispatch after dispatch has no return flag behind it, so the layer must synchronise and meet
    the other ranks on the host first; the usual dispatch -> combine -> dispatch order must not."""
    from amd_distributed_2025_b200.models import moe_all2all as m

    calls = []

    class Engine:
        def dispatch(self, x, idx):
            calls.append("dispatch")
            return 0

        def combine(self, out, w, y):
            calls.append("combine")
            return 0

    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: calls.append("sync"))
    monkeypatch.setattr(m.dist, "is_initialized", lambda: True)
    monkeypatch.setattr(m.dist, "barrier", lambda group=None: calls.append("barrier"))
    layer = m.MoEAllToAll.__new__(m.MoEAllToAll)
    cfg = contract.MoEConfig(num_experts=8, experts_per_token=2, hidden_dim=16, max_num_tokens=4,
                             in_dtype=torch.float32, out_dtype=torch.float32)
    layer.cfg, layer.world_size, layer.rank, layer.group, layer.device = cfg, 2, 0, None, torch.device("cpu")
    layer.engine, layer.monitor, layer._dispatch_pending, layer._num_tokens = Engine(), None, False, 0
    layer.ws = type("W", (), {"check": lambda self, sync=True: None})()
    layer.expert_num_tokens = layer.expert_x = layer.expert_meta = None
    layer.expert_y = torch.zeros(4, 8, 16)
    x, idx, w = torch.zeros(4, 16), torch.zeros(4, 2, dtype=torch.int32), torch.zeros(4, 2)
    y = torch.zeros(4, 16)
    layer.dispatch(x, idx)
    layer.combine(y, w, None, layer.expert_y, None)
    layer.dispatch(x, idx)
    assert calls == ["dispatch", "combine", "dispatch"]
    layer.dispatch(x, idx)  # no combine in between
    assert calls[3:] == ["sync", "barrier", "dispatch"]
    layer.world_size = 1
    layer.dispatch(x, idx)  # a single rank has no peers to wait for
    assert calls[6:] == ["dispatch"]
