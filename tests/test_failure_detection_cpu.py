"""Failure detection on the host (CPU ranks, no GPU involved): a rank that leaves between
steps, a rank whose heartbeat stops, and a rank that never joins."""
import datetime
import multiprocessing as mp
import os
import time

import torch
import torch.distributed as dist

from amd_distributed_2025_b200.harness.eval import free_port, run_ranks


def _leave_between_steps(rank, world_size):
    from amd_distributed_2025_b200.parallel.health import HealthMonitor, PeerLostError, default_store

    mon = HealthMonitor(default_store(), rank, world_size, stale_after_s=30.0)
    dist.barrier()
    steps_done = 0

    def step():
        t = torch.ones(4)
        dist.all_reduce(t)
        return float(t[0])

    assert mon.guarded(step) == world_size
    steps_done += 1
    dist.barrier()
    if rank == world_size - 1:
        mon.leave("planned exit after step 1")
        return {"left": True, "steps": steps_done}
    # the survivors learn about it on the host, before launching the next collective
    deadline = time.time() + 20
    while time.time() < deadline:
        try:
            mon.guarded(lambda: None)
        except PeerLostError as err:
            return {"left": False, "steps": steps_done, "lost": err.ranks}
        time.sleep(0.05)
    return {"left": False, "steps": steps_done, "lost": []}


def test_rank_leaving_between_steps_is_seen_before_next_launch():
    res = run_ranks(_leave_between_steps, 3, "gloo", (), 120.0)
    assert res[2]["left"]
    for r in res[:2]:
        assert r["lost"] == [2] and r["steps"] == 1


def _stale_heartbeat(rank, world_size):
    from amd_distributed_2025_b200.parallel.health import HealthMonitor, PeerLostError, default_store

    mon = HealthMonitor(default_store(), rank, world_size, stale_after_s=0.5)
    dist.barrier()
    if rank == 1:
        time.sleep(2.0)  # alive but silent: no heartbeats
        dist.barrier()
        return {"lost": None}
    lost = []
    deadline = time.time() + 10
    while time.time() < deadline and not lost:
        mon.beat()
        try:
            mon.assert_all_alive()
        except PeerLostError as err:
            lost = err.ranks
        time.sleep(0.1)
    dist.barrier()
    return {"lost": lost}


def test_stale_heartbeat_is_reported():
    res = run_ranks(_stale_heartbeat, 2, "gloo", (), 120.0)
    assert res[0]["lost"] == [1]


def _never_joined(port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        # world of 2, but rank 1 is never started: rendezvous must fail, not hang
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        q.put("joined")
    except Exception as exc:  # noqa: BLE001
        q.put(type(exc).__name__)


def test_rank_that_never_joins_fails_rendezvous_within_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_never_joined, args=(free_port(), q))
    t0 = time.time()
    p.start()
    p.join(60)
    assert not p.is_alive()
    assert q.get(timeout=5) != "joined"
    assert time.time() - t0 < 60


def _operator_sees_departure(rank, world_size):
    """The shared-memory operators consult the monitor themselves: after a rank has left between
    steps, the survivors' next operator call raises ``PeerLostError`` on the host instead of
    waiting for the departed rank's flags."""
    from amd_distributed_2025_b200 import contract
    from amd_distributed_2025_b200.models.host_ops import HostGemmRS, HostMoEAllToAll
    from amd_distributed_2025_b200.parallel.health import HealthMonitor, PeerLostError, default_store

    mon = HealthMonitor(default_store(), rank, world_size, stale_after_s=60.0)
    cfg, data, _, _ = contract.make_moe_inputs(6, 2, 32, 8, 5, rank, world_size, device="cpu", dtype=torch.float32,
                                               fixed_num_tokens=8)
    layer = HostMoEAllToAll(cfg, rank, world_size, wait_limit_ms=20000, monitor=mon)
    op = HostGemmRS(6 * 16 * 4, rank, world_size, wait_limit_ms=20000, monitor=mon)
    a, w, bias = contract.make_gemm_rs_inputs(rank, world_size, 6, 16, 24, True, 3, device="cpu")
    a, w, bias = a.float(), w.float(), bias.float()
    y = layer.forward(data.x, data.indices, data.weights, 1 + rank)  # step 1: everybody is there
    op(a, w, bias)
    dist.barrier()
    out = {"step1": list(y.shape), "left": False, "moe": None, "gemm": None}
    if rank == world_size - 1:
        mon.leave("planned exit after step 1")
        out["left"] = True
    else:
        deadline = time.time() + 20
        while time.time() < deadline and out["moe"] is None:
            try:
                mon.assert_all_alive()
                time.sleep(0.05)
                continue
            except PeerLostError:
                pass
            try:
                layer.forward(data.x, data.indices, data.weights, 1 + rank)
                out["moe"] = "no error"
            except PeerLostError as err:
                out["moe"] = err.ranks
            try:
                op(a, w, bias)
                out["gemm"] = "no error"
            except PeerLostError as err:
                out["gemm"] = err.ranks
    dist.barrier()
    layer.close()
    op.close()
    return out


def test_shared_memory_operators_raise_peer_lost_from_the_call_itself():
    res = run_ranks(_operator_sees_departure, 3, "gloo", (), 180.0)
    assert res[2]["left"]
    for r in res[:2]:
        assert r["moe"] == [2] and r["gemm"] == [2], r
