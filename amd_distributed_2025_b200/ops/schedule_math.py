"""Host restatements of the index arithmetic inside the kernels, for tests and for reading.

Nothing here runs on a hot path.  Each function states, in plain Python, what a kernel
computes with warps and flags, so that CPU tests can pin the arithmetic:

* ``dispatch_slots`` -- the slot every ``(token, k)`` entry gets in its owner's expert buffer
  (csrc/moe_kernels.cu): rows of lower source ranks first (the exchanged count matrix), then
  this rank's earlier entries with the same expert.  This is the reference's row order
  (all2all/reference.py:79-86, 107-112, 140-146).
* ``dedup_dispatch`` / ``dedup_combine`` -- the de-duplicating protocol of csrc/moe_dedup.cu with
  the large kernel's partition of the tokens over CTAs and warps: per-warp histograms, prefix
  over warps and CTAs, one landed row per (token, destination rank), per-(source, token) row
  lists on the owner, replication into the expert buffers, and the owner-side weighted
  pre-reduction with one returned row per (source, token).
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


def dedup_dispatch(indices_per_rank: Sequence[Sequence[Sequence[int]]], num_experts: int, max_recv: int,
                   grid: int = 3, warps: int = 8):
    """The dedup dispatch as the large kernel partitions it: CTA ``b`` of ``grid`` owns tokens
    ``[b * tpc, (b + 1) * tpc)``, its warp ``w`` a contiguous part of them.  Returns per owner rank
    ``(meta, tok_rows, landed)``: ``meta[row] = (expert, src, token, k)``, ``tok_rows[(src, t)]`` the
    k-list of final rows on that owner (or -1), ``landed`` the set of ``(src, t)`` that crossed to it."""
    ws = len(indices_per_rank)
    e_local = num_experts // ws
    counts = [[0] * num_experts for _ in range(ws)]
    per_rank = []
    for r, idx in enumerate(indices_per_rank):
        n_tok = len(idx)
        tpc = -(-n_tok // grid) if n_tok else 0
        tpw = -(-tpc // warps) if tpc else 0
        whist = [[[0] * num_experts for _ in range(warps)] for _ in range(grid)]
        ranges = {}
        for b in range(grid):
            c0, c1 = min(n_tok, b * tpc), min(n_tok, b * tpc + tpc)
            for w in range(warps):
                t0 = min(c1, c0 + w * tpw)
                t1 = min(c1, t0 + tpw)
                ranges[(b, w)] = (t0, t1)
                for t in range(t0, t1):
                    for e in idx[t]:
                        whist[b][w][e] += 1
        blk = [[sum(whist[b][w][e] for w in range(warps)) for e in range(num_experts)] for b in range(grid)]
        for e in range(num_experts):
            counts[r][e] = sum(blk[b][e] for b in range(grid))
        per_rank.append((whist, blk, ranges))
    owners = [({}, {}, set()) for _ in range(ws)]
    for r, idx in enumerate(indices_per_rank):
        whist, blk, ranges = per_rank[r]
        for b in range(grid):
            base = [sum(blk[g][e] for g in range(b)) + sum(counts[s][e] for s in range(r)) for e in range(num_experts)]
            for w in range(warps):
                run = [sum(whist[b][v][e] for v in range(w)) for e in range(num_experts)]  # exclusive prefix over warps
                t0, t1 = ranges[(b, w)]
                for t in range(t0, t1):
                    rows = []
                    for kk, e in enumerate(idx[t]):
                        slot = base[e] + run[e]
                        run[e] += 1
                        dst = e // e_local
                        row = (e % e_local) * max_recv + slot if slot < max_recv else -1
                        rows.append((dst, row))
                        if row >= 0:
                            owners[dst][0][row] = (e, r, t, kk)
                    for d in {dst for dst, _ in rows}:
                        owners[d][1][(r, t)] = [row if dst == d else -1 for dst, row in rows]
                        if d != r:
                            owners[d][2].add((r, t))
    return counts, owners


def dedup_combine(owners, weights_per_rank, expert_y_per_rank, num_tokens: Sequence[int], hidden: int):
    """Owner-side pre-reduction and source-side sum: ``out[src][t] = sum over owners d (ascending) of
    sum over the entries of (src, t) on d (ascending k) of w * expert_y[d][row]``; plain floats."""
    ws = len(owners)
    out = [[[0.0] * hidden for _ in range(num_tokens[r])] for r in range(ws)]
    for d in range(ws):
        _, tok_rows, _ = owners[d]
        for (src, t), rows in sorted(tok_rows.items()):
            part = [0.0] * hidden
            for kk, row in enumerate(rows):
                if row < 0:
                    continue
                w = weights_per_rank[src][t][kk]
                y = expert_y_per_rank[d][row]
                for h in range(hidden):
                    part[h] += w * y[h]
            for h in range(hidden):
                out[src][t][h] += part[h]
    return out


def dedup_chunk_tokens_sender(num_tokens: int, grid: int, chunks: int, warps: int = 8) -> List[List[int]]:
    """Tokens a source rank sends under DATA-flag value ``c + 1``, for every chunk ``c``: each warp
    cuts ITS OWN contiguous token range ``[t0, t1)`` into ``chunks`` parts, part ``c`` being
    ``[t0 + ceil(c * len / C), t0 + ceil((c + 1) * len / C))`` (``moe_dedup_dispatch_kernel``,
    landing loop)."""
    out: List[List[int]] = [[] for _ in range(chunks)]
    tpc = -(-num_tokens // grid)
    tpw = -(-tpc // warps)
    for b in range(grid):
        c0 = min(num_tokens, b * tpc)
        c1 = min(num_tokens, c0 + tpc)
        for w in range(warps):
            t0 = min(c1, c0 + w * tpw)
            t1 = min(c1, t0 + tpw)
            n = t1 - t0
            for c in range(chunks):
                out[c].extend(range(t0 + (c * n + chunks - 1) // chunks, t0 + ((c + 1) * n + chunks - 1) // chunks))
    return out


def dedup_chunk_tokens_receiver(num_tokens: int, grid: int, chunks: int, chunk: int, pieces: int = 1,
                                warps: int = 8) -> List[Tuple[int, int]]:
    """(token, piece) items an owner rank replicates for chunk ``chunk`` of a source that announced
    ``(num_tokens, grid, chunks)`` in its info word: the dense numbering ``(source warp, position in
    its share of the chunk, piece)`` of the replication loop.  ``grid == 0`` (the small kernel's
    announcement) counts as one CTA."""
    gs = max(grid, 1)
    tpc = -(-num_tokens // gs)
    tpw = -(-tpc // warps)
    max_sub = -(-tpw // chunks)
    items: List[Tuple[int, int]] = []
    for item in range(gs * warps * max_sub * pieces):
        piece = item % pieces
        q = item // pieces
        sub = q % max_sub
        pair = q // max_sub
        g, w = divmod(pair, warps)
        n = min(tpw, min(tpc, num_tokens - g * tpc) - w * tpw)
        if n <= 0:
            continue
        i = (chunk * n + chunks - 1) // chunks + sub
        if i >= ((chunk + 1) * n + chunks - 1) // chunks:
            continue
        items.append((g * tpc + w * tpw + i, piece))
    return items


def gemm_reduce_work(m: int, n: int, world_size: int, rank: int, block_n: int, grid: int, fuse_own: bool,
                     splits: int = 1, warps_per_cta: int = 11, block_m: int = 128, epilogue_warps: int = 4):
    """The reduction work of ``gemm_rs_kernel``'s reducer warps on one rank, as ``reduce_staged_units``
    enumerates it: the staged m-blocks of this rank's rows, cut into units (whole tiles or 32-row
    quarters), units into ``cuts`` runs of 8-column vectors, work items dealt to the CTAs round robin
    (CTA ``b`` starts at ``grid - 1 - b``).  Returns ``(items, cuts, parts)`` with ``items`` a list of
    ``(cta, row, first_vector, vectors)`` spans -- one per (unit, cut, row) -- for coverage checks."""
    rows_per_rank = m // world_size
    row_lo = rank * rows_per_rank
    n_tiles = -(-n // block_n)
    mb_lo, mb_hi = row_lo // block_m, (row_lo + rows_per_rank - 1) // block_m

    def owned(mb: int) -> bool:
        lo = mb * block_m
        return (fuse_own and splits == 1 and lo >= row_lo and lo + block_m <= row_lo + rows_per_rank
                and lo + block_m <= m)

    lo_staged = not owned(mb_lo)
    hi_staged = mb_hi != mb_lo and not owned(mb_hi)
    all_staged = not (fuse_own and splits == 1)
    n_mb = (mb_hi - mb_lo + 1) if all_staged else int(lo_staged) + int(hi_staged)
    if n_mb == 0:
        return [], 0, 0
    parts = 1 if n_mb * n_tiles >= 2 * grid else epilogue_warps
    rows_per_part = block_m // parts
    total_units = n_tiles * n_mb * parts
    unit_items = rows_per_part * (block_n // 8)
    cuts = (2 * grid * warps_per_cta + total_units - 1) // total_units
    cuts = max(1, min(cuts, unit_items // 128, 16))
    cut_items = -(-unit_items // cuts)
    total_work = total_units * cuts
    items = []
    for cta in range(grid):
        j = grid - 1 - cta
        while j < total_work:
            cut, unit = j % cuts, j // cuts
            part, rest = unit % parts, unit // parts
            mi, nb = rest % n_mb, rest // n_mb
            mb = mb_lo + mi if all_staged else (mb_lo if (mi == 0 and lo_staged) else mb_hi)
            r0 = max(mb * block_m + part * rows_per_part, row_lo)
            r1 = min(mb * block_m + (part + 1) * rows_per_part, row_lo + rows_per_rank, m)
            if r1 > r0:
                c0 = nb * block_n
                c1 = min(c0 + block_n, n)
                vec_per_row = (c1 - c0) >> 3
                n_items = (r1 - r0) * vec_per_row
                lo, hi = cut * cut_items, min(n_items, (cut + 1) * cut_items)
                i = lo
                while i < hi:
                    row, v = divmod(i, vec_per_row)
                    run = min(hi - i, vec_per_row - v)
                    items.append((cta, r0 + row, (c0 >> 3) + v, run))
                    i += run
            j += grid
    return items, cuts, parts
