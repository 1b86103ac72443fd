"""Decoding of the status words written by device kernels (csrc/status.h).

The reference has no failure reporting: a rank that never arrives hangs the collective
(all2all/hipv8.py:281).  Kernels here bound every wait and leave a record instead.
"""
from __future__ import annotations

STATUS_CODES = {0: "ok", 1: "timeout", 2: "bad_index", 3: "bad_argument"}
PHASES = {
    0: "none",
    1: "grid_barrier",
    2: "moe_counts",
    3: "moe_data",
    4: "moe_y_ready",
    5: "rs_partials",
    6: "gemm_pipeline",
    7: "barrier",
    8: "selftest",
    9: "moe_weights",
    10: "moe_return",
}


class StatusError(RuntimeError):
    """A device kernel gave up on a wait or skipped an out-of-range access."""

    def __init__(self, message: str, status: dict):
        super().__init__(message)
        self.status = dict(status)

    @property
    def code(self) -> str:
        return STATUS_CODES.get(self.status.get("code", -1), "unknown")

    @property
    def phase(self) -> str:
        return PHASES.get(self.status.get("phase", -1), "unknown")


def describe_status(st: dict, rank: int = -1) -> str:
    code = STATUS_CODES.get(st.get("code", -1), f"code {st.get('code')}")
    phase = PHASES.get(st.get("phase", -1), f"phase {st.get('phase')}")
    return (
        f"rank {rank}: device kernel reported {code} in phase {phase} "
        f"(peer {st.get('peer')}, detail {st.get('detail')}, epoch {st.get('epoch')}, last seen {st.get('seen')})"
    )
