"""Failure detection on GPUs, in the forms that cannot hurt a shared device: a rank leaves
BETWEEN steps with nothing in flight and stays alive (so its memory stays mapped) until the test
is over.  The survivor either learns about it on the host before its next launch (monitor), or
launches anyway and its kernel's bounded wait runs out and leaves a status record; the CUDA
context stays usable either way.  NVLS is off in every library used, and the kernels under
test use plain peer stores."""
import os

import pytest
import torch

from amd_distributed_2025_b200 import contract, oracle
from amd_distributed_2025_b200.harness.eval import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _departure(rank, world_size):
    import torch.distributed as dist

    from amd_distributed_2025_b200.models import moe_all2all
    from amd_distributed_2025_b200.parallel.health import HealthMonitor, PeerLostError, default_store
    from amd_distributed_2025_b200.utils.status import StatusError

    dev = torch.device("cuda", torch.cuda.current_device())
    store = default_store()
    mon = HealthMonitor(store, rank, world_size, stale_after_s=120.0)
    cfg, data, _, _ = contract.make_moe_inputs(16, 2, 512, 32, 9, rank, world_size, device=dev, fixed_num_tokens=32)
    watched = moe_all2all.MoEAllToAll(cfg, rank, world_size, wait_limit_ms=50, monitor=mon)  # consults the monitor
    blind = moe_all2all.MoEAllToAll(cfg, rank, world_size, wait_limit_ms=50)                 # does not
    out = {"rank": rank}
    for layer in (watched, blind):  # step 1 on both layers: everybody is there
        y = layer.forward(data.x, data.indices, data.weights, 1 + rank)
        torch.cuda.synchronize()
        layer.check()
        ok, _ = oracle.check_moe_output(y, oracle.moe_expected_output(cfg, data, world_size))
        out.setdefault("step1_ok", True)
        out["step1_ok"] = out["step1_ok"] and bool(ok)
    dist.barrier()
    if rank == world_size - 1:
        # leave between steps: nothing of this rank is in flight; the process stays until the others are done
        torch.cuda.synchronize()
        mon.leave("planned exit after step 1")
        store.wait(["test/survivors_done"])
    else:
        store.wait([f"b200/health/left/{world_size - 1}"])
        if rank == 0:
            try:  # (a) noticed on the host, nothing is launched
                watched.forward(data.x, data.indices, data.weights, 1 + rank)
                out["host_notice"] = "no error"
            except PeerLostError as err:
                out["host_notice"] = err.ranks
            try:  # (b) launched anyway: the kernel's wait for the departed rank's counts runs out
                blind.forward(data.x, data.indices, data.weights, 1 + rank)
                torch.cuda.synchronize()
                blind.check()
                out["device_wait"] = "no error"
            except StatusError as err:
                out["device_wait"] = [err.code, err.phase, err.status["peer"]]
            # the context is intact: a single-rank layer works
            cfg1, d1, _, _ = contract.make_moe_inputs(8, 2, 256, 16, 4, 0, 1, device=dev, fixed_num_tokens=16)
            solo = moe_all2all.MoEAllToAll(cfg1, 0, 1)
            y1 = solo.forward(d1.x, d1.indices, d1.weights, 1.0)
            torch.cuda.synchronize()
            solo.check()
            ok1, _ = oracle.check_moe_output(y1, oracle.moe_expected_output(cfg1, d1, 1))
            out["context_usable"] = bool(ok1)
            solo.close()
            store.set("test/survivors_done", "1")
        else:
            store.wait(["test/survivors_done"])
    dist.barrier()
    blind.ws.reset_status()
    watched.close(collective=True)
    blind.close(collective=True)
    return out


def test_departed_rank_is_noticed_on_the_host_or_by_a_bounded_device_wait():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"  # inherited by the spawned ranks
    res = run_ranks(_departure, 2, "nccl", (), 300.0)
    assert all(r["step1_ok"] for r in res)
    r0 = res[0]
    assert r0["host_notice"] == [1]
    assert r0["device_wait"] == ["timeout", "moe_counts", 1]
    assert r0["context_usable"]
