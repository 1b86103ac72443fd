"""The signalling protocol of the symmetric heap, exercised by CPU processes on a
host-shared-memory stand-in: epochs instead of resets, payload visibility after a flag,
a peer that signals late, a peer that never signals, a peer that has exited."""
import multiprocessing as mp
import os
import time

import pytest
import torch

HEADER = 4096


def _heap(prefix, rank, ws, nbytes=HEADER + 4096):
    from amd_distributed_2025_b200.ops import _ext

    ext = _ext.load()
    heap = ext.HostShmHeap(prefix, rank, ws, nbytes)
    assert heap.open_peers(20_000_000_000)
    return ext, heap


def _ring_worker(prefix, rank, ws, rounds, q):
    try:
        ext, heap = _heap(prefix, rank, ws)
        assert heap.barrier(1, 10_000_000_000)["code"] == 0
        nxt, prv = (rank + 1) % ws, (rank - 1) % ws
        ok = True
        for epoch in range(1, rounds + 1):
            # payload first, then the flag (release); the reader waits (acquire), then reads
            heap.view(nxt, HEADER, [4], torch.int64).copy_(torch.tensor([rank, epoch, epoch * 7 + rank, 0]))
            heap.signal(ext.FLAG_TEST, nxt, epoch)
            st = heap.wait(ext.FLAG_TEST, prv, epoch, 10_000_000_000)
            got = heap.view(rank, HEADER, [4], torch.int64).tolist()
            ok = ok and st["code"] == 0 and got[:3] == [prv, epoch, epoch * 7 + prv]
            # nobody overwrites a payload before its reader is done: barrier per round, epoch-numbered
            assert heap.barrier(1 + epoch, 10_000_000_000)["code"] == 0
        q.put((rank, ok))
        heap.close()
    except Exception as exc:  # noqa: BLE001
        q.put((rank, repr(exc)))


def test_epoch_flags_carry_payload_around_a_ring():
    ws, prefix = 3, f"b200t_ring_{os.getpid()}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ring_worker, args=(prefix, r, ws, 50, q)) for r in range(ws)]
    [p.start() for p in procs]
    res = dict(q.get(timeout=120) for _ in range(ws))
    [p.join(30) for p in procs]
    assert res == {0: True, 1: True, 2: True}


def _silent_peer_worker(prefix, rank, ws, mode, q):
    try:
        ext, heap = _heap(prefix, rank, ws)
        assert heap.barrier(1, 10_000_000_000)["code"] == 0
        if rank == 1:
            if mode == "late":
                time.sleep(0.3)
                heap.signal(ext.FLAG_TEST, 0, 5)
            elif mode == "exit":
                q.put((rank, "left"))
                heap.close()
                return
            # mode == "never": simply does not signal
            time.sleep(1.0)
            q.put((rank, "done"))
            heap.close()
            return
        t0 = time.time()
        st = heap.wait(ext.FLAG_TEST, 1, 5, 2_000_000_000 if mode == "late" else 200_000_000)
        took = time.time() - t0
        # the process is fine afterwards: the status can be read, cleared, and the heap reused
        first = heap.status()
        heap.reset_status()
        q.put((rank, {"st": st, "took": took, "first": first, "cleared": heap.status()["code"]}))
        heap.close()
    except Exception as exc:  # noqa: BLE001
        q.put((rank, repr(exc)))


@pytest.mark.parametrize("mode", ["late", "never", "exit"])
def test_bounded_wait_on_a_late_silent_or_departed_peer(mode):
    ws, prefix = 2, f"b200t_{mode}_{os.getpid()}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_silent_peer_worker, args=(prefix, r, ws, mode, q)) for r in range(ws)]
    [p.start() for p in procs]
    res = dict(q.get(timeout=60) for _ in range(ws))
    [p.join(30) for p in procs]
    r0 = res[0]
    assert isinstance(r0, dict), r0
    if mode == "late":
        assert r0["st"]["code"] == 0 and 0.2 < r0["took"] < 2.0
    else:
        st = r0["st"]
        assert st["code"] == 1 and st["peer"] == 1 and st["epoch"] == 5 and st["seen"] == 0  # timeout, who, what
        assert 0.15 < r0["took"] < 5.0
        assert r0["first"]["code"] == 1 and r0["cleared"] == 0
