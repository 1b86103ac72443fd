"""Symmetric workspaces for CPU ranks of one node (POSIX shared memory).

The CPU counterpart of ``symm_mem.SymmetricWorkspace``: one slab per rank with the same
header of epoch-numbered flags, mapped by every rank, over ``HostShmHeap``
(csrc/host_shm_heap.h).  The operators in ``models/host_ops.py`` run the device kernels'
protocols on it.  The reference's ranks meet only inside library collectives
(all2all/reference.py:91-119, gemm-rs/reference.py:59); nothing here calls one after set-up.

Set-up needs a name that all ranks agree on and nobody else uses: ``shared_prefix`` draws
one on rank 0 and sends it through the process group, or the caller passes its own.
"""
from __future__ import annotations

import os
import socket
import time
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..utils.status import StatusError, describe_status
from .symm_mem import DEFAULT_WAIT_LIMIT_MS, EpochCounter, SlabLayout

_counter = 0
_single_node: dict = {}


def single_node(group=None) -> bool:
    """True when every rank of ``group`` runs on this machine (one exchange per group, cached)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return True
    key = id(group)
    if key not in _single_node:
        try:
            with open("/proc/sys/kernel/random/boot_id", "r", encoding="ascii") as fh:
                ident = fh.read().strip()
        except OSError:
            ident = ""
        ident = f"{socket.gethostname()}/{ident}"
        names = [None] * dist.get_world_size(group)
        dist.all_gather_object(names, ident, group=group)
        _single_node[key] = len(set(names)) == 1
    return _single_node[key]


def shared_prefix(group=None, tag: str = "ws") -> str:
    """A shared-memory name prefix unique to this call, identical on all ranks of ``group``."""
    global _counter
    _counter += 1
    name = [f"b200_{tag}_{os.getpid()}_{_counter}_{time.time_ns() & 0xFFFFFF:x}"]
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast_object_list(name, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    return name[0]


class HostSymmetricWorkspace:
    """A slab in shared memory per rank, with layout, epochs and bounded waits."""

    def __init__(
        self,
        layout: SlabLayout,
        prefix: str,
        rank: int,
        world_size: int,
        wait_limit_ms: Optional[float] = None,
        open_limit_ms: float = 30000.0,
    ):
        from ..ops import _ext

        self.ext = _ext.load()
        if world_size > self.ext.MAX_WORLD_SIZE:
            raise ValueError(f"world_size {world_size} exceeds the supported {self.ext.MAX_WORLD_SIZE}")
        self.rank, self.world_size = rank, world_size
        self.layout = layout
        self.epochs = EpochCounter()
        self.wait_limit_ns = int((wait_limit_ms if wait_limit_ms is not None else DEFAULT_WAIT_LIMIT_MS) * 1e6)
        self.heap = self.ext.HostShmHeap(prefix, rank, world_size, layout.total_bytes)
        if not self.heap.open_peers(int(open_limit_ms * 1e6)):
            self.heap.close()
            raise StatusError(
                f"rank {rank}: a peer's shared-memory slab {prefix!r} did not appear within {open_limit_ms:.0f} ms",
                {"code": 1, "phase": 0, "peer": -1, "detail": 0, "epoch": 0, "seen": 0},
            )
        self._closed = False
        # everyone has mapped everything once this barrier is through: drop the names, so that a
        # rank that dies later leaves no segment behind
        self.barrier()
        self.heap.unlink()

    def view(self, name: str, shape: Sequence[int], dtype: torch.dtype, rank: Optional[int] = None) -> torch.Tensor:
        """Tensor over a region of rank ``rank``'s slab (default: the own one); no copy."""
        off, size = self.layout.regions[name]
        need = torch.empty((), dtype=dtype).element_size()
        for s in shape:
            need *= int(s)
        if need > size:
            raise ValueError(f"view of {need} bytes exceeds region {name!r} of {size} bytes")
        return self.heap.view(self.rank if rank is None else rank, off, list(shape), dtype)

    def offset(self, name: str) -> int:
        return self.layout.offset(name)

    def next_epoch(self, name: str) -> int:
        return self.epochs.next(name)

    def raise_on(self, status: dict) -> None:
        if status["code"] != 0:
            raise StatusError(describe_status(status, self.rank).replace("device kernel", "host operator"), status)

    def barrier(self) -> None:
        self.raise_on(self.heap.barrier(self.next_epoch("barrier"), self.wait_limit_ns))

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            self.heap.close()
