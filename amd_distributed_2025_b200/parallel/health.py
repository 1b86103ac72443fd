"""Host-side failure detection for ranks that share symmetric workspaces.

The reference has none: a rank that dies leaves its peers inside a library collective
forever (all2all/hipv8.py:281).  The kernels here bound their own waits (csrc/signal.cuh),
and this module adds the host half: every rank posts heartbeats and an explicit
"leaving" note on a key-value store, and checks the board *before* launching a kernel
that will wait on peers.  A peer that left, or whose heartbeat is stale, turns the next
launch into a ``PeerLostError`` on the host instead of an expired wait on the device.

Ranks must leave only between steps, with none of their kernels in flight.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional



class PeerLostError(RuntimeError):
    def __init__(self, message: str, ranks: List[int]):
        super().__init__(message)
        self.ranks = list(ranks)


class HealthMonitor:
    def __init__(self, store, rank: int, world_size: int, prefix: str = "b200/health", stale_after_s: float = 10.0):
        self.store = store
        self.rank = rank
        self.world_size = world_size
        self.prefix = prefix
        self.stale_after_s = stale_after_s
        self.beat()

    # -- this rank ---------------------------------------------------------------------
    def beat(self) -> None:
        self.store.set(f"{self.prefix}/beat/{self.rank}", repr(time.time()))

    def leave(self, reason: str = "left") -> None:
        """Announce an orderly departure; call with no kernels in flight."""
        self.store.set(f"{self.prefix}/left/{self.rank}", reason)

    # -- the others --------------------------------------------------------------------
    def _get(self, key: str) -> Optional[str]:
        if not self.store.check([key]):
            return None
        return self.store.get(key).decode()

    def departed(self) -> Dict[int, str]:
        out = {}
        for r in range(self.world_size):
            v = self._get(f"{self.prefix}/left/{r}")
            if v is not None:
                out[r] = v
        return out

    def stale(self, now: Optional[float] = None) -> List[int]:
        now = time.time() if now is None else now
        out = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            v = self._get(f"{self.prefix}/beat/{r}")
            if v is None or now - float(v) > self.stale_after_s:
                out.append(r)
        return out

    def assert_all_alive(self) -> None:
        gone = {r: why for r, why in self.departed().items() if r != self.rank}
        if gone:
            raise PeerLostError(f"rank {self.rank}: peers left the job: {gone}", sorted(gone))
        old = self.stale()
        if old:
            raise PeerLostError(f"rank {self.rank}: no heartbeat from ranks {old} for {self.stale_after_s} s", old)

    def guarded(self, fn: Callable, *args, **kwargs):
        """Heartbeat, verify the peers, then run ``fn`` (a launch that waits on peers)."""
        self.beat()
        self.assert_all_alive()
        return fn(*args, **kwargs)


def default_store():
    """The store of the default process group."""
    from torch.distributed import distributed_c10d

    return distributed_c10d._get_default_store()
