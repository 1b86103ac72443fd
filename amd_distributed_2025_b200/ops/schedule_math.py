"""Host restatements of the index arithmetic inside the kernels, for tests and for reading.

Nothing here runs on a hot path.  Each function states, in plain Python, what a kernel
computes with warps and flags, so that CPU tests can pin the arithmetic:

* ``dispatch_slots`` -- the slot every ``(token, k)`` entry gets in its owner's expert buffer
  (csrc/moe_kernels.cu): rows of lower source ranks first (the exchanged count matrix), then
  this rank's earlier entries with the same expert.  This is the reference's row order
  (all2all/reference.py:79-86, 107-112, 140-146).
* ``gemm_tile_order`` -- the order in which a CTA (pair) scheduler of ``gemm_rs_kernel`` visits
  its work items: K slices innermost, column tiles inside a band of row groups, bands along
  the row-group sequence that is rotated so the rank's own rows come last
  (csrc/gemm_rs_sm100.cu: ``tile_coords``, ``launch_typed``).
* ``gemm_tile_owners`` / ``expected_arrivals`` -- who owns the rows of a 128-row block and how
  many arrivals the owner's per-(tile, quarter) counter must see.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

BLOCK_M = 128


def dispatch_slots(indices_per_rank: Sequence[Sequence[Sequence[int]]], num_experts: int) -> Tuple[List[List[int]], List[Dict[Tuple[int, int], Tuple[int, int, int]]]]:
    """``indices_per_rank[r][t][k]`` -> (count matrix ``[src][expert]``, per source rank a map
    ``(t, k) -> (owner rank, local expert, slot)``)."""
    ws = len(indices_per_rank)
    e_local = num_experts // ws
    counts = [[0] * num_experts for _ in range(ws)]
    for r, idx in enumerate(indices_per_rank):
        for row in idx:
            for e in row:
                counts[r][e] += 1
    routes: List[Dict[Tuple[int, int], Tuple[int, int, int]]] = []
    for r, idx in enumerate(indices_per_rank):
        seen = [0] * num_experts  # this rank's earlier entries per expert, in (t, k) order
        route = {}
        for t, row in enumerate(idx):
            for k, e in enumerate(row):
                src_prefix = sum(counts[s][e] for s in range(r))
                route[(t, k)] = (e // e_local, e % e_local, src_prefix + seen[e])
                seen[e] += 1
        routes.append(route)
    return counts, routes


def gemm_tile_order(m: int, n: int, world_size: int, rank: int, block_n: int, ctas: int, splits: int = 1) -> List[Tuple[int, int, int]]:
    """Work items ``(row group, column tile, K slice)`` in the order scheduler 0 of a grid with ONE
    scheduler would visit them (scheduler ``g`` of ``G`` takes items ``g, g + G, ...``)."""
    m_tiles = -(-m // BLOCK_M)
    n_tiles = -(-n // block_n)
    m_groups = -(-m_tiles // ctas)
    rows_per_rank = m // world_size
    group_rows = BLOCK_M * ctas
    m_start = (-(-((rank + 1) * rows_per_rank) // group_rows)) % m_groups
    groups_per_rank = max(rows_per_rank // group_rows, 1)
    band = max(1, min(8, groups_per_rank, m_groups))
    order = []
    for tile in range(m_groups * n_tiles):
        per_band = band * n_tiles
        b = tile // per_band
        start = b * band
        size = min(band, m_groups - start)
        within = tile - start * n_tiles
        nb = within // size
        mg = (m_start + start + (within - nb * size)) % m_groups
        for s in range(splits):
            order.append((mg, nb, s))
    return order


def gemm_tile_owners(m: int, world_size: int, block: int) -> List[int]:
    """Ranks that own at least one row of 128-row block ``block`` (empty past the end of M)."""
    rows_per_rank = m // world_size
    lo = block * BLOCK_M
    hi = min(m, lo + BLOCK_M) - 1
    if hi < lo:
        return []
    return list(range(lo // rows_per_rank, hi // rows_per_rank + 1))


def block_is_own(m: int, world_size: int, rank: int, block: int) -> bool:
    """True when every row of the block belongs to ``rank`` -- the tiles a rank may finish in its
    own epilogue."""
    rows_per_rank = m // world_size
    lo = block * BLOCK_M
    return lo >= rank * rows_per_rank and lo + BLOCK_M <= (rank + 1) * rows_per_rank and lo + BLOCK_M <= m


def expected_arrivals(world_size: int, splits: int, fused_own: bool) -> int:
    """Arrivals per (tile, 32-row quarter) counter: every (virtual) rank once, minus this rank when
    it keeps its own partial in registers."""
    return world_size - 1 if (fused_own and splits == 1) else world_size * splits
