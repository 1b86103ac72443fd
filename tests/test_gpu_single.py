"""Single-GPU tests: every kernel at world_size 1 against plain PyTorch fp32/fp64 math."""
import pytest
import torch

from amd_distributed_2025_b200 import contract, oracle

pytestmark = pytest.mark.gpu


def _ext():
    from amd_distributed_2025_b200.ops import _ext

    return _ext.load()


def test_extension_is_loaded_from_tree():
    mod = _ext()
    assert mod.__file__.endswith("_C/b200_ext.so")


def test_bounded_wait_times_out_and_context_survives():
    from amd_distributed_2025_b200.parallel.symm_mem import SlabLayout, SymmetricWorkspace
    from amd_distributed_2025_b200.utils.status import StatusError

    ext = _ext()
    ws = SymmetricWorkspace(SlabLayout(ext.HEAP_HEADER_BYTES), rank=0, world_size=1, wait_limit_ms=5)
    ws.check(sync=True)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    ws.heap.wait_selftest(3, 12345, 5_000_000)  # a flag nothing sets, 5 ms limit
    stop.record()
    torch.cuda.synchronize()
    assert 4.0 < start.elapsed_time(stop) < 500.0
    with pytest.raises(StatusError) as err:
        ws.check(sync=True)
    assert err.value.code == "timeout" and err.value.phase == "selftest" and err.value.status["peer"] == 3
    assert ws.status()["code"] == 1  # host mirror, no synchronisation needed
    ws.reset_status()
    ws.check(sync=True)
    # the context is still usable
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
    ws.barrier()
    torch.cuda.synchronize()
    ws.check(sync=True)
    ws.close()


@pytest.mark.parametrize("mode", ["dedup", "direct"])
@pytest.mark.parametrize(
    "E,k,H,T,dtype,fixed",
    [
        (8, 2, 6144, 4, torch.float16, None),
        (64, 6, 2048, 8, torch.float16, None),
        (128, 4, 2880, 32, torch.float16, None),
        (256, 8, 7168, 128, torch.bfloat16, 128),
        (16, 2, 256, 32, torch.float32, 32),
        (64, 6, 1024, 1024, torch.bfloat16, 1024),  # > 4096 entries: the grid-barrier kernels
        (256, 8, 512, 600, torch.float16, 600),
        (8, 2, 250, 5, torch.float16, 5),  # row size not a multiple of 16 bytes: scalar paths
    ],
)
def test_moe_world1_matches_oracle(E, k, H, T, dtype, fixed, mode):
    from amd_distributed_2025_b200.models import moe_all2all

    for it in range(3):  # new inputs (and token counts) every call: nothing of the previous call may survive
        n_tok = None if fixed is None else max(fixed - 3 * it, 1)
        cfg, data, rank, ws = contract.make_moe_inputs(E, k, H, T, 7 + it, 0, 1, device="cuda", dtype=dtype,
                                                       fixed_num_tokens=n_tok, routing="zipf" if T >= 600 else "uniform",
                                                       weights="softmax")
        layer = moe_all2all.get_layer(cfg, 0, 1, mode=mode)
        if it == 1:
            got = layer.dispatch(data.x, data.indices)
            torch.cuda.synchronize()
            layer.check()
            ok, msg = oracle.compare_dispatch_layout(got, oracle.moe_dispatch_oracle(cfg, [data], 0))
            assert ok, msg
            layer.expert_scale(1.0)
            y = torch.empty(data.num_tokens, H, dtype=dtype, device="cuda")
            layer.combine(y, data.weights, got[2], layer.expert_y, got[0], data.num_tokens)
        else:
            y = moe_all2all.custom_kernel((cfg, data, 0, 1), mode=mode)
        torch.cuda.synchronize()
        layer.check()
        ok, msg = oracle.check_moe_output(y, oracle.moe_expected_output(cfg, data, 1))
        assert ok, (it, msg)
        assert oracle.relative_error(y, oracle.moe_expected_output(cfg, data, 1, acc_dtype=torch.float64)) < 5e-3


def test_moe_dedup_fp32_partial_rows_and_phase_stamps():
    from amd_distributed_2025_b200.models import moe_all2all

    cfg, data, _, _ = contract.make_moe_inputs(32, 4, 1024, 96, 11, 0, 1, device="cuda", dtype=torch.bfloat16,
                                               fixed_num_tokens=96, weights="softmax")
    layer = moe_all2all.MoEAllToAll(cfg, 0, 1, mode="dedup", partial_dtype=torch.float32)
    layer.enable_trace()
    y = layer.forward(data.x, data.indices, data.weights, 1.0)
    torch.cuda.synchronize()
    layer.check()
    ok, msg = oracle.check_moe_output(y, oracle.moe_expected_output(cfg, data, 1))
    assert ok, msg
    d, c = layer.trace[0].tolist(), layer.trace[1].tolist()
    assert all(v > 0 for v in d) and d[:7] == sorted(d[:7]) and d[7] >= d[6]  # dispatch phases in order
    assert c[0] > 0 and c[7] >= c[2] >= c[1] >= c[0] and c[0] >= d[0]
    layer.close()


@pytest.mark.parametrize("mode", ["dedup", "direct"])
def test_moe_combine_accepts_foreign_expert_y(mode):
    from amd_distributed_2025_b200.models import moe_all2all

    cfg, data, _, _ = contract.make_moe_inputs(32, 4, 512, 64, 3, 0, 1, device="cuda", fixed_num_tokens=64)
    layer = moe_all2all.get_layer(cfg, 0, 1, mode=mode)
    n_tok, ex, em = layer.dispatch(data.x, data.indices)
    ey = ex.clone() * 3  # an ordinary tensor, not the symmetric buffer
    y = torch.zeros(cfg.max_num_tokens, cfg.hidden_dim, dtype=cfg.out_dtype, device="cuda")
    layer.combine(y, data.weights, em, ey, n_tok, data.num_tokens)
    torch.cuda.synchronize()
    want = (data.x.float() * 3 * data.weights.sum(1, keepdim=True)).to(cfg.out_dtype)
    assert torch.allclose(y[: data.num_tokens].float(), want.float(), rtol=1e-2, atol=5e-3)


@pytest.mark.parametrize("mode", ["dedup", "direct"])
def test_moe_bad_expert_id_is_reported_not_faulted(mode):
    from amd_distributed_2025_b200.models import moe_all2all
    from amd_distributed_2025_b200.utils.status import StatusError

    cfg, data, _, _ = contract.make_moe_inputs(16, 2, 128, 8, 3, 0, 1, device="cuda", fixed_num_tokens=8)
    layer = moe_all2all.MoEAllToAll(cfg, 0, 1, mode=mode)
    bad = data.indices.clone()
    bad[2, 1] = 99
    y = layer.forward(data.x, bad, data.weights, 2.0)
    torch.cuda.synchronize()
    with pytest.raises(StatusError) as err:
        layer.check()
    assert err.value.code == "bad_index"
    # the other entries were served: every token but the one with the bad id has its full result
    want = (data.x.float() * 2 * data.weights.sum(1, keepdim=True)).to(cfg.out_dtype)
    keep = [t for t in range(8) if t != 2]
    assert torch.allclose(y[keep].float(), want[keep].float(), rtol=1e-2, atol=5e-3)
    layer.ws.reset_status()
    layer.close()


@pytest.mark.parametrize(
    "m,n,k,has_bias",
    [
        (128, 256, 64, False),      # one tile, one k-block
        (128, 256, 512, True),
        (256, 512, 1024, True),
        (64, 2880, 360, True),      # ragged M, N and K (K/8 of the smallest task shape)
        (2048, 5120, 1600, True),
        (512, 4608, 4608, False),
        (1024, 8192, 3584, True),
    ],
)
def test_gemm_world1_matches_fp32_reference(m, n, k, has_bias):
    from amd_distributed_2025_b200.models import gemm_rs

    a, w, bias = contract.make_gemm_rs_inputs(0, 1, m, n, k, has_bias, 5, device="cuda")
    out = gemm_rs.custom_kernel((a, w, bias))
    torch.cuda.synchronize()
    gemm_rs.get_op(m, n, k).check()
    truth = a.float() @ w.float().T
    if has_bias:
        truth = truth + bias.float()
    want = oracle.gemm_rs_fused_rounding([a], [w], bias, 0)
    assert oracle.outlier_fraction(out, want, oracle.GEMM_RS_RTOL, oracle.GEMM_RS_ATOL) < 1e-4
    assert oracle.relative_error(out, truth) < 5e-3


@pytest.mark.parametrize("m,n,k,has_bias", [(64, 2880, 360, True), (512, 4096, 1536, True), (2048, 2880, 360, True)])
def test_gemm_world1_reference_inputs_pass_reference_checker(m, n, k, has_bias):
    """Operands from the reference generator (uniform +-0.01) against the library path."""
    from amd_distributed_2025_b200.models import gemm_rs

    a, w, bias = contract.generate_gemm_rs_input(0, 1, m, n, k, has_bias, 2035, device="cuda")
    out = gemm_rs.custom_kernel((a, w, bias))
    ref = torch.matmul(a, w.T) + bias
    ok, msg = oracle.check_gemm_rs_output(out, ref)
    assert ok, msg
    truth = a.double() @ w.double().T + bias.double()
    assert oracle.relative_error(out, truth) < 5e-3


@pytest.mark.parametrize("block_n,cta_pair,splits",
                         [(64, 0, 1), (128, 0, 1), (256, 0, 1), (128, 1, 1), (192, 1, 1), (256, 1, 1),
                          (256, 1, 3), (192, 1, 2), (128, 0, 4)])
@pytest.mark.parametrize("m,n,k", [(384, 1024, 832), (128, 256, 64), (1000, 2880, 360), (2048, 2048, 2048)])
def test_gemm_tile_shapes_single_cta_and_cta_pair(block_n, cta_pair, splits, m, n, k):
    """Every tile width, as single CTAs and as CTA pairs (256-row tiles, odd block counts
    and ragged edges included), gives the same GEMM."""
    from amd_distributed_2025_b200.models import gemm_rs

    a, w, bias = contract.make_gemm_rs_inputs(0, 1, m, n, k, True, 9, device="cuda")
    if splits > (k + 63) // 64:
        pytest.skip("more K slices than k-blocks")
    op = gemm_rs.get_op(m, n, k)
    op.block_n, op.cta_pair, op.splits = block_n, cta_pair, splits
    try:
        for _ in range(3):  # staged paths alternate parities and reset their counters
            out = op(a, w, bias)
        torch.cuda.synchronize()
        op.check()
    finally:
        op.block_n, op.cta_pair, op.splits = 0, -1, 0
    truth = a.float() @ w.float().T + bias.float()
    assert oracle.relative_error(out, truth) < 5e-3
    want = oracle.gemm_rs_fused_rounding([a], [w], bias, 0)
    assert oracle.outlier_fraction(out, want, oracle.GEMM_RS_RTOL, oracle.GEMM_RS_ATOL) < 1e-4


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (1000, 2944, 1024), (4096, 4096, 2048)])
def test_fp8_block_scaled_gemm_matches_fp32_reference(m, n, k):
    from amd_distributed_2025_b200.ops.fp8_gemm import fp8_gemm, fp8_gemm_reference

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
    kb, nb = (k + 127) // 128, (n + 127) // 128
    # scales stored the way the stand-alone template indexes them: [kb][m] and [kb][nb], viewed transposed
    a_scale = (torch.rand(kb, m, device="cuda", generator=g) + 0.5).t()
    b_scale = (torch.rand(kb, nb, device="cuda", generator=g) + 0.5).t()
    c = fp8_gemm(a, b, a_scale, b_scale)
    torch.cuda.synchronize()
    want = fp8_gemm_reference(a, b, a_scale, b_scale)
    assert oracle.relative_error(c, want) < 5e-3
    assert torch.allclose(c.float(), want, rtol=2e-2, atol=2e-2 * float(want.abs().max()))


@pytest.mark.parametrize("tma_store", [True, False])
@pytest.mark.parametrize("fuse_own", [True, False])
@pytest.mark.parametrize("m,n,k,block_n,cta_pair", [(2048, 2048, 1024, 256, 1), (1024, 2880, 512, 192, 1), (512, 1024, 256, 128, 0),
                                                   (1056, 1000, 320, 256, 1)])
def test_gemm_staged_path_on_one_gpu(tma_store, fuse_own, m, n, k, block_n, cta_pair):
    """The multi-rank machinery (staging buffer, TMA stores, signaller, arrival counters,
    reduction) run on a single rank, where its result must equal the plain GEMM."""
    from amd_distributed_2025_b200.models import gemm_rs

    a, w, bias = contract.make_gemm_rs_inputs(0, 1, m, n, k, True, 13, device="cuda")
    op = gemm_rs.get_op(m, n, k)
    op.block_n, op.cta_pair, op.splits = block_n, cta_pair, 1
    op.force_staged, op.tma_store, op.fuse_own = True, tma_store, fuse_own
    try:
        for _ in range(3):
            out = op(a, w, bias)
        torch.cuda.synchronize()
        op.check()
    finally:
        op.block_n, op.cta_pair, op.splits = 0, -1, 0
        op.force_staged, op.tma_store, op.fuse_own = False, True, None
    want = oracle.gemm_rs_fused_rounding([a], [w], bias, 0)
    assert oracle.outlier_fraction(out, want, oracle.GEMM_RS_RTOL, oracle.GEMM_RS_ATOL) < 1e-4
    assert oracle.relative_error(out, a.float() @ w.float().T + bias.float()) < 5e-3
