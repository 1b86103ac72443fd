"""Symmetric workspaces: peer-mapped device memory plus the host side of its protocol.

The reference has no such layer: ranks exchange data only through
``torch.distributed`` collectives on ordinary tensors (all2all/hipv8.py:281-359,
gemm-rs/reference.py:59).  Here a ``SymmetricWorkspace`` is one slab per rank with the
same layout everywhere.  Creation is collective: every rank allocates, the CUDA IPC
handles travel once through the existing process group (``all_gather_object``), every
rank maps the peers' slabs, and a host barrier closes the set-up.  Afterwards kernels
reach "offset X on rank r" with plain loads/stores over NVLink and synchronise through
epoch-numbered flags in the slab header; the process group is not used again.

``SlabLayout`` is the pure-Python bump allocator that assigns the offsets; because it is
deterministic, all ranks derive identical layouts without communicating.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..utils.status import StatusError, describe_status

DEFAULT_WAIT_LIMIT_MS = float(os.environ.get("B200_WAIT_LIMIT_MS", "10000"))
CANARY_BYTE = 0xA5


def checked() -> bool:
    """``B200_CHECKED=1`` selects the checked flavour: guard words between the regions of
    every slab (verified by ``check()``), and range checks before every remote store of the
    GEMM epilogue.  It stands in for a memory sanitizer, which the reference does not use
    either (its guards are the hand-written range checks of all2all/hipv8.py:118,124,198,205)."""
    return os.environ.get("B200_CHECKED", "0").strip() not in ("", "0", "false", "False")


def checked_guard_bytes() -> int:
    return 1024 if checked() else 0


def _align_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class SlabLayout:
    """Deterministic bump allocator over one slab; offsets are bytes from the slab base."""

    def __init__(self, header_bytes: int, align: int = 1024, guard_bytes: int = 0):
        self.align = align
        self.cursor = _align_up(header_bytes, align)
        self.regions: Dict[str, Tuple[int, int]] = {}
        self.guard_bytes = int(guard_bytes)
        self.guards: List[Tuple[int, int]] = []  # (offset, bytes) of the canary areas after each region

    def add(self, name: str, nbytes: int, align: Optional[int] = None) -> int:
        if name in self.regions:
            raise KeyError(f"region {name!r} already allocated")
        a = align or self.align
        off = _align_up(self.cursor, a)
        self.regions[name] = (off, int(nbytes))
        self.cursor = off + int(nbytes)
        if self.guard_bytes:
            # a canary area right behind the region: an overrun of the region lands here first
            g = _align_up(self.cursor, 16)
            self.guards.append((g, self.guard_bytes))
            self.cursor = g + self.guard_bytes
        return off

    def offset(self, name: str) -> int:
        return self.regions[name][0]

    def size(self, name: str) -> int:
        return self.regions[name][1]

    @property
    def total_bytes(self) -> int:
        return _align_up(self.cursor, self.align)

    def overlaps(self) -> bool:
        spans = sorted(self.regions.values())
        return any(a_off + a_len > b_off for (a_off, a_len), (b_off, _) in zip(spans, spans[1:]))


class EpochCounter:
    """Call numbers per protocol.  Flags carry the epoch of the call that set them, so
    they never need resetting; all ranks must issue the same sequence of calls."""

    def __init__(self):
        self._epochs: Dict[str, int] = {}

    def next(self, name: str) -> int:
        v = self._epochs.get(name, 0) + 1
        self._epochs[name] = v
        return v

    def current(self, name: str) -> int:
        return self._epochs.get(name, 0)


class SymmetricWorkspace:
    """A peer-mapped slab with its layout, epochs and status word."""

    def __init__(
        self,
        layout: SlabLayout,
        *,
        rank: Optional[int] = None,
        world_size: Optional[int] = None,
        group=None,
        device: Optional[torch.device] = None,
        wait_limit_ms: Optional[float] = None,
        poison_on_timeout: bool = False,
        heap=None,
    ):
        from ..ops import _ext

        # A protocol whose flags do not carry the call number (the arrival counters of the fused
        # GEMM) cannot be trusted after an expired wait: late arrivals of the failed call would
        # satisfy the next one.  Such a workspace stays poisoned until recover() is run collectively.
        self.poison_on_timeout = bool(poison_on_timeout)
        self.poisoned: Optional[dict] = None
        self._canary_views: List[torch.Tensor] = []
        if heap is not None:
            # pre-built heap (tests drive the host-side state machine with a stand-in)
            self.ext, self.group, self.heap = None, group, heap
            self.world_size, self.rank = world_size or 1, rank or 0
            self.device, self.layout, self.epochs = device, layout, EpochCounter()
            self.wait_limit_ns = int((wait_limit_ms if wait_limit_ms is not None else DEFAULT_WAIT_LIMIT_MS) * 1e6)
            self._closed = False
            return
        self.ext = _ext.load()
        self.group = group
        initialized = dist.is_available() and dist.is_initialized()
        self.world_size = world_size if world_size is not None else (dist.get_world_size(group) if initialized else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if initialized else 0)
        if self.world_size > self.ext.MAX_WORLD_SIZE:
            raise ValueError(f"world_size {self.world_size} exceeds the supported {self.ext.MAX_WORLD_SIZE}")
        if self.world_size > 1 and not initialized:
            raise RuntimeError("a process group is required to exchange memory handles")
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = torch.device(device)
        self.layout = layout
        self.epochs = EpochCounter()
        self.wait_limit_ns = int((wait_limit_ms if wait_limit_ms is not None else DEFAULT_WAIT_LIMIT_MS) * 1e6)
        dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.heap = self.ext.SymmHeap(self.rank, self.world_size, layout.total_bytes, dev_index)
        if self.world_size > 1:
            handles: List[Optional[bytes]] = [None] * self.world_size
            dist.all_gather_object(handles, self.heap.ipc_handle(), group=group)
            self.heap.open_peers(handles)
            dist.barrier(group=group)
        self._closed = False
        for off, nbytes in layout.guards:
            view = self.heap.view(off, [nbytes], torch.uint8)
            view.fill_(CANARY_BYTE)
            self._canary_views.append(view)

    # -- memory ------------------------------------------------------------------------
    def view(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """Tensor view of a region of the *local* slab (no copy; lifetime = workspace)."""
        off, size = self.layout.regions[name]
        need = int(torch.tensor([], dtype=dtype).element_size())
        for s in shape:
            need *= int(s)
        if need > size:
            raise ValueError(f"view of {need} bytes exceeds region {name!r} of {size} bytes")
        return self.heap.view(off, list(shape), dtype)

    def offset(self, name: str) -> int:
        return self.layout.offset(name)

    # -- protocol ----------------------------------------------------------------------
    def next_epoch(self, name: str) -> int:
        return self.epochs.next(name)

    def barrier(self) -> None:
        """Device-side barrier over all ranks on the current stream."""
        self.heap.barrier(self.next_epoch("barrier"), self.wait_limit_ns)

    def status(self, sync: bool = False) -> dict:
        return self.heap.status_sync() if sync else self.heap.status()

    def check(self, sync: bool = False) -> None:
        """Raise ``StatusError`` if a kernel recorded a failure (expired wait, bad index), or if
        an earlier expired wait poisoned the workspace (see ``recover``)."""
        if self.poisoned is not None:
            raise StatusError(
                describe_status(self.poisoned, self.rank) + "; the workspace stays unusable until recover() "
                "has been called by all ranks together", self.poisoned)
        if not sync and self.heap.status_code() == 0:
            return
        st = self.status(sync)
        if st["code"] != 0:
            if self.poison_on_timeout and st["code"] == 1 and self.world_size > 1:
                self.poisoned = dict(st)
            raise StatusError(describe_status(st, self.rank), st)

    def reset_status(self) -> None:
        """Clear the status record.  Does not lift a poisoning: that takes ``recover``."""
        self.heap.reset_status()

    def recover(self, zero_regions: Sequence[str] = ()) -> None:
        """Collective recovery after an expired wait: every rank drains its stream, the ranks
        meet on the host, each zeroes the named regions of its own slab (arrival counters) and
        its status record, the call numbers restart, and the ranks meet again before anybody
        launches.  All surviving ranks of the group must call it."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        initialized = dist.is_available() and dist.is_initialized()
        if self.world_size > 1 and initialized:
            dist.barrier(group=self.group)
        for name in zero_regions:
            off, size = self.layout.regions[name]
            self.heap.view(off, [size], torch.uint8).zero_()
        self.heap.reset_status()
        self.epochs = EpochCounter()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if self.world_size > 1 and initialized:
            dist.barrier(group=self.group)
        self.poisoned = None

    def check_canaries(self) -> None:
        """With guard areas (``B200_CHECKED=1``): raise if any byte behind a region changed."""
        for (off, nbytes), view in zip(self.layout.guards, self._canary_views):
            if not bool((view == CANARY_BYTE).all()):
                bad = int((view != CANARY_BYTE).nonzero()[0])
                name = next((n for n, (o, sz) in self.layout.regions.items() if o + sz <= off < o + sz + 32), "?")
                raise StatusError(f"rank {self.rank}: guard area behind region {name!r} was overwritten "
                                  f"(first bad byte at slab offset {off + bad})", {"code": 2, "phase": 0, "peer": -1,
                                                                                 "detail": off + bad, "epoch": 0, "seen": 0})

    def close(self, collective: bool = False) -> None:
        """Release the slab.  With ``collective=True`` (all ranks call it together, idle) the
        peers' mappings are dropped first and the ranks meet on the host before anybody frees
        its slab, so no slab is freed while a peer still maps it."""
        if self._closed:
            return
        self._closed = True
        if collective and self.world_size > 1 and dist.is_initialized():
            self.heap.close_peers()
            dist.barrier(group=self.group)
        self.heap.close()


class McastWorkspace:
    """A region of device memory per rank, all bound into one NVLink multicast object (NVLS).

    ``local`` views address this rank's own memory; ``mc_ptr`` is the multicast address, through
    which ``multimem.ld_reduce`` returns sums formed inside NVSwitch.  Creation and ``close`` are
    collective.  ``McastWorkspace.probe`` tells whether the device and driver offer multicast at
    all; creation can still fail (no permission to pass descriptors between the ranks, no switch):
    callers treat any exception as "not available here" and keep their peer-to-peer path.

    A rank must not exit while its memory is bound and peers may still read through the
    multicast address: call ``close(collective=True)`` on every rank while idle.  The reference
    has no counterpart (its reduce-scatter is a library call, gemm-rs/reference.py:59).
    """

    @staticmethod
    def probe(device: Optional[int] = None) -> Tuple[bool, str]:
        from ..ops import _ext

        ext = _ext.load()
        dev = torch.cuda.current_device() if device is None else device
        ok, why = ext.McastRegion.supported(dev)
        return bool(ok), str(why)

    def __init__(self, nbytes: int, *, rank: Optional[int] = None, world_size: Optional[int] = None, group=None):
        from ..ops import _ext

        ext = _ext.load()
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("a process group is required to share the multicast object")
        self.group = group
        self.world_size = world_size if world_size is not None else dist.get_world_size(group)
        self.rank = rank if rank is not None else dist.get_rank(group)
        dev = torch.cuda.current_device()
        # every step is followed by an agreement on its outcome, so that no rank is left waiting for
        # a peer that gave up
        self.region = None
        err = ""
        try:
            self.region = ext.McastRegion(self.rank, self.world_size, int(nbytes), dev)
        except Exception as exc:  # noqa: BLE001
            err = str(exc)
        self._agree(err, "creating the region")
        fd, err = -1, ""
        if self.rank == 0:
            try:
                fd = self.region.create_and_export()
            except Exception as exc:  # noqa: BLE001
                err = str(exc)
        shared: List[Optional[tuple]] = [None] * self.world_size
        dist.all_gather_object(shared, (os.getpid(), fd, err), group=group)
        root_pid, root_fd, root_err = shared[0]
        if root_err:
            self._fail(f"rank 0 could not create the multicast object: {root_err}")
        err = ""
        if self.rank != 0:
            try:
                self.region.import_from(root_pid, root_fd)
            except Exception as exc:  # noqa: BLE001
                err = str(exc)
        self._agree(err, "importing the multicast object")
        err = ""
        try:
            self.region.add_device()
        except Exception as exc:  # noqa: BLE001
            err = str(exc)
        self._agree(err, "adding the devices")  # also the barrier the driver wants before any bind
        err = ""
        try:
            self.region.bind_and_map()
        except Exception as exc:  # noqa: BLE001
            err = str(exc)
        self._agree(err, "binding and mapping")
        self.bytes = self.region.bytes
        self._closed = False

    def _agree(self, err: str, what: str) -> None:
        errs: List[Optional[str]] = [None] * self.world_size
        dist.all_gather_object(errs, err, group=self.group)
        bad = {r: e for r, e in enumerate(errs) if e}
        if bad:
            self._fail(f"{what} failed on ranks {sorted(bad)}: {next(iter(bad.values()))}")

    def _fail(self, message: str) -> None:
        if self.region is not None:
            try:
                self.region.close()
            except Exception:  # noqa: BLE001
                pass
            self.region = None
        raise RuntimeError("NVLink multicast is not available here: " + message)

    @property
    def mc_ptr(self) -> int:
        return self.region.mc_ptr

    @property
    def local_ptr(self) -> int:
        return self.region.local_ptr

    def view(self, offset: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        return self.region.view(offset, list(shape), dtype)

    def close(self, collective: bool = True) -> None:
        if self._closed or self.region is None:
            return
        self._closed = True
        torch.cuda.synchronize()
        if collective:
            dist.barrier(group=self.group)  # nobody reads through the multicast address any more
        self.region.close()
        if collective:
            dist.barrier(group=self.group)
