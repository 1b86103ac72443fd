"""CPU tests pinning the index arithmetic the kernels implement (slot assignment of dispatch,
tile order and ownership of the fused GEMM)."""
import itertools

import pytest
import torch

from amd_distributed_2025_b200 import contract, oracle
from amd_distributed_2025_b200.contract import MoEConfig, RankTestData
from amd_distributed_2025_b200.ops import schedule_math as sm


@pytest.mark.parametrize("ws,E,k,T", [(1, 8, 2, 5), (2, 16, 2, 32), (4, 64, 6, 8), (8, 256, 8, 16)])
def test_dispatch_slots_reproduce_the_oracle_layout(ws, E, k, T):
    cfg = MoEConfig(E, k, 8, T, torch.float32, torch.float32)
    data = []
    for r in range(ws):
        g = torch.Generator().manual_seed(100 + r)
        data.append(RankTestData(cfg, g, r, device="cpu", fixed_num_tokens=T if r % 2 == 0 else max(T - 3, 0)))
    counts, routes = sm.dispatch_slots([d.indices.tolist() for d in data], E)
    e_local = E // ws
    for owner in range(ws):
        n_tok, _, meta = oracle.moe_dispatch_oracle(cfg, data, owner)
        # expert_num_tokens = column sums of the count matrix over the owner's experts
        assert n_tok.tolist() == [sum(counts[s][owner * e_local + el] for s in range(ws)) for el in range(e_local)]
        for el in range(e_local):
            for slot in range(int(n_tok[el])):
                e, src, t, kk = meta[el, slot, :4].tolist()
                assert routes[src][(t, kk)] == (owner, el, slot)
    # every slot of an expert is used exactly once
    for owner in range(ws):
        used = sorted((el, slot) for r in routes for (o, el, slot) in r.values() if o == owner)
        assert len(used) == len(set(used))


@pytest.mark.parametrize("m,n,ws,block_n,ctas,splits",
                         [(8192, 8192, 8, 256, 2, 1), (8192, 8192, 1, 256, 2, 1), (2048, 5120, 8, 192, 2, 1),
                          (256, 5120, 8, 128, 2, 1), (256, 5120, 1, 256, 2, 3), (64, 7168, 8, 256, 1, 4),
                          (4096, 2880, 4, 256, 2, 1), (1000 // 8 * 8, 2880, 2, 128, 1, 1)])
def test_gemm_tile_order_covers_everything_once_and_ends_with_own_rows(m, n, ws, block_n, ctas, splits):
    m_tiles, n_tiles = -(-m // 128), -(-n // block_n)
    m_groups = -(-m_tiles // ctas)
    for rank in range(ws):
        order = sm.gemm_tile_order(m, n, ws, rank, block_n, ctas, splits)
        assert sorted(order) == sorted(itertools.product(range(m_groups), range(n_tiles), range(splits)))
        # the row groups that hold this rank's rows are the last ones visited
        rows = m // ws
        own_groups = {b // ctas for b in range(m_tiles) if rank in sm.gemm_tile_owners(m, ws, b)
                      and (rank * rows <= b * 128 or ws == 1 or rows < 128 * ctas)}
        seq = [mg for mg, _, _ in order]
        first_own = min(i for i, mg in enumerate(seq) if mg in own_groups)
        if rows % (128 * ctas) == 0 and ws > 1:
            assert all(mg in own_groups for mg in seq[first_own:])
        # K slices of one tile are adjacent (they run concurrently on neighbouring schedulers)
        for i in range(0, len(order), splits):
            assert len({(mg, nb) for mg, nb, _ in order[i : i + splits]}) == 1


def test_ownership_and_arrival_counts():
    # 8 ranks x 1024 rows: blocks 0..7 are rank 0's, all of them wholly owned
    assert sm.gemm_tile_owners(8192, 8, 0) == [0] and sm.gemm_tile_owners(8192, 8, 8) == [1]
    assert sm.block_is_own(8192, 8, 1, 8) and not sm.block_is_own(8192, 8, 0, 8)
    # 8 ranks x 32 rows: one 128-row block holds four owners, nobody owns it wholly
    assert sm.gemm_tile_owners(256, 8, 1) == [4, 5, 6, 7]
    assert not any(sm.block_is_own(256, 8, r, 1) for r in range(8))
    # ragged end: M = 64 has half a block, a block past the end has no owner
    assert sm.gemm_tile_owners(64, 8, 0) == list(range(8)) and sm.gemm_tile_owners(64, 8, 1) == []
    assert sm.expected_arrivals(8, 1, fused_own=True) == 7
    assert sm.expected_arrivals(8, 1, fused_own=False) == 8
    assert sm.expected_arrivals(2, 3, fused_own=True) == 6  # K slices are always staged


@pytest.mark.parametrize("ws,E,k,T,grid", [(1, 8, 2, 9, 3), (2, 16, 2, 37, 4), (4, 64, 6, 21, 2), (8, 64, 6, 40, 5)])
def test_dedup_protocol_reproduces_oracle_layout_and_output(ws, E, k, T, grid):
    """One landed row per (token, destination rank), replicated by the owner, gives the oracle's
    dispatch layout; owner-side pre-reduced rows summed by the source give the oracle's output."""
    H = 4
    cfg = MoEConfig(E, k, H, T, torch.float32, torch.float32)
    data = []
    for r in range(ws):
        g = torch.Generator().manual_seed(7 + r)
        data.append(RankTestData(cfg, g, r, device="cpu", fixed_num_tokens=T if r % 2 == 0 else max(T - 5, 0)))
    max_recv = cfg.max_recv(ws)
    counts, owners = sm.dedup_dispatch([d.indices.tolist() for d in data], E, max_recv, grid=grid)
    e_local = E // ws
    expert_y = []
    for owner in range(ws):
        n_tok, ex, meta = oracle.moe_dispatch_oracle(cfg, data, owner)
        got_meta, tok_rows, landed = owners[owner]
        rows = {el * max_recv + s: tuple(meta[el, s, :4].tolist()) for el in range(e_local) for s in range(int(n_tok[el]))}
        assert got_meta == rows
        # replication: every final row is fed by the landed (or local) row of its (src, token)
        for (src, t), lst in tok_rows.items():
            assert (src, t) in landed or src == owner
            for kk, row in enumerate(lst):
                if row >= 0:
                    assert torch.equal(ex.reshape(-1, H)[row], data[src].x[t]) and rows[row][1:] == (src, t, kk)
        # a token lands at most once per destination: that is the whole point
        assert len(landed) == len({(s, t) for (s, t) in tok_rows if s != owner})
        expert_y.append((ex.reshape(-1, H) * (1 + owner)).tolist())
    out = sm.dedup_combine(owners, [d.weights.tolist() for d in data], expert_y, [d.num_tokens for d in data], H)
    for r in range(ws):
        want = oracle.moe_expected_output(cfg, data[r], ws)
        assert torch.allclose(torch.tensor(out[r], dtype=torch.float32).reshape(-1, H), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("chunks", [1, 2, 3, 4, 7, 8])
def test_dedup_chunks_sender_and_receiver_enumerate_the_same_tokens(chunks):
    """What a source sends under chunk flag c must be exactly what the owner replicates after
    seeing that flag, for token counts that divide neither the grid, the warps nor the chunks."""
    for grid in (1, 2, 3, 37, 148, 296):
        for tokens in (0, 1, 2, 7, 8, 9, 63, 64, 65, 127, 1000, 1023, 1024, 4095, 4096, 4097):
            sent = sm.dedup_chunk_tokens_sender(tokens, grid, chunks)
            assert sorted(t for part in sent for t in part) == list(range(tokens)), (tokens, grid, chunks)
            for c in range(chunks):
                for pieces in (1, 4):
                    got = sm.dedup_chunk_tokens_receiver(tokens, grid, chunks, c, pieces=pieces)
                    assert len(set(got)) == len(got)
                    assert sorted(got) == sorted((t, p) for t in sent[c] for p in range(pieces)), (tokens, grid, chunks, c)


def test_dedup_small_kernel_announcement_covers_every_token():
    """The small kernel announces grid 0 and one chunk: the owner must still visit tokens 0..T-1."""
    for tokens in (0, 1, 5, 128, 511, 512):
        got = sm.dedup_chunk_tokens_receiver(tokens, 0, 1, 0)
        assert sorted(t for t, _ in got) == list(range(tokens))


def _task_gemm_shapes():
    from amd_distributed_2025_b200 import contract

    shapes = {(s["m"], s["n"], s["k"]) for name in ("tests", "benchmarks") for s in contract.task_specs("gemm_rs", name)}
    return sorted(shapes | {(8192, 8192, 28672), (2048, 5120, 12800), (256, 5120, 12800)})


@pytest.mark.parametrize("world_size", [1, 2, 4, 8])
def test_gemm_reducers_cover_every_staged_output_vector_exactly_once(world_size):
    """Units, cuts and the round-robin deal of ``reduce_staged_units``: for every task shape, plan
    and grid, the staged rows of a rank (all of them above 4 ranks or with K slices, else the partly
    owned m-blocks) are reduced once each, and every CTA gets within one work item of its share."""
    from amd_distributed_2025_b200.ops import _ext

    ext = _ext.load()
    for m, n, k in _task_gemm_shapes():
        if m % world_size or (k // world_size) < 64:
            continue
        plan = ext.gemm_rs_plan(m, n, k // world_size, world_size, 0, -1, 0)
        bn, splits = plan["block_n"], plan["splits"]
        fuse_own = world_size <= 4
        rows = m // world_size
        for grid in (148, 74, 5):
            for rank in sorted({0, world_size // 2, world_size - 1}):
                items, cuts, parts = sm.gemm_reduce_work(m, n, world_size, rank, bn, grid, fuse_own, splits)
                seen = {}
                per_cta = [0] * grid
                for cta, row, v0, run in items:
                    per_cta[cta] += run
                    for v in range(v0, v0 + run):
                        seen[(row, v)] = seen.get((row, v), 0) + 1
                assert all(c == 1 for c in seen.values()), (m, n, k, world_size, grid, rank)
                row_lo = rank * rows
                expect_rows = []
                for row in range(row_lo, row_lo + rows):
                    lo = (row // 128) * 128
                    tile_owned = (fuse_own and splits == 1 and lo >= row_lo and lo + 128 <= row_lo + rows and lo + 128 <= m)
                    if not tile_owned:
                        expect_rows.append(row)
                assert len(seen) == len(expect_rows) * (n // 8), (m, n, k, world_size, grid, rank, cuts, parts)
                assert {r for r, _ in seen} == set(expect_rows)
                assert 1 <= cuts <= 16 or not items
