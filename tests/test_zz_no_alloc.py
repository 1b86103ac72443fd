"""The allocation-free dispatch entry point, called through its exported C symbol.

Some users of this library cannot let it allocate: their process has already given the
whole device to its own pool, or they sit in a loop where a cudaMalloc would stall the
GPU.  ``b200_moe_dispatch_noalloc`` serves them: it takes the caller's buffers and keeps
its intermediates in a fixed array inside the library.  This test feeds it the same
inputs as the regular ``MoEAllToAll.dispatch`` (world size 1) and demands identical
results, twice in a row with different inputs, because the second call starts from
whatever the first left in the shared array.
"""
import ctypes

import pytest
import torch

from amd_distributed_2025_b200 import contract

pytestmark = pytest.mark.gpu


def _lib():
    from amd_distributed_2025_b200.ops import _ext

    mod = _ext.load()
    lib = ctypes.CDLL(mod.__file__)
    fn = lib.b200_moe_dispatch_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.b200_moe_dispatch_noalloc_error.restype = ctypes.c_char_p
    lib.b200_moe_dispatch_noalloc_status.restype = ctypes.c_int
    return lib


def _run_both(lib, layer, cfg, data, out):
    """Regular entry point, then the C symbol on the same inputs; returns both results."""
    n_ref, x_ref, m_ref = layer.dispatch(data.x, data.indices)
    torch.cuda.synchronize()
    layer.check()
    ref = (n_ref.clone(), x_ref.clone(), m_ref.clone(), layer._route[: data.num_tokens * cfg.experts_per_token].clone())

    ex, em, en, route = out
    idx = data.indices.to(torch.int32).contiguous()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.b200_moe_dispatch_noalloc(
        data.x.data_ptr(), idx.data_ptr(), data.num_tokens, cfg.experts_per_token,
        cfg.hidden_dim * data.x.element_size(), cfg.num_experts, cfg.max_num_tokens,
        ex.data_ptr(), em.data_ptr(), en.data_ptr(), route.data_ptr(),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    assert rc == 0, lib.b200_moe_dispatch_noalloc_error().decode()
    assert lib.b200_moe_dispatch_noalloc_status() == 0
    moved = free_before - torch.cuda.mem_get_info()[0]  # device memory taken while the C call ran
    return ref, (en, ex, em, route[: data.num_tokens * cfg.experts_per_token]), moved


def _assert_same(cfg, ref, got):
    n_ref, x_ref, m_ref, r_ref = ref
    n_got, x_got, m_got, r_got = got
    assert torch.equal(n_ref, n_got)
    assert torch.equal(r_ref, r_got)
    for e, n in enumerate(n_ref.tolist()):
        assert torch.equal(x_ref[e, :n], x_got[e, :n])
        assert torch.equal(m_ref[e, :n], m_got[e, :n])


def test_noalloc_dispatch_matches_regular_entry_point_twice():
    from amd_distributed_2025_b200.models import moe_all2all

    lib = _lib()
    E, k, H, T = 64, 6, 2048, 96
    cfg, first, _, _ = contract.make_moe_inputs(E, k, H, T, 17, 0, 1, device="cuda", fixed_num_tokens=T)
    _, second, _, _ = contract.make_moe_inputs(E, k, H, T, 99, 0, 1, device="cuda", fixed_num_tokens=T - 29,
                                               routing="zipf")
    layer = moe_all2all.MoEAllToAll(cfg, 0, 1)
    out = (
        torch.zeros(E, T, H, dtype=cfg.in_dtype, device="cuda"),
        torch.zeros(E, T, 5, dtype=torch.int32, device="cuda"),
        torch.zeros(E, dtype=torch.int32, device="cuda"),
        torch.zeros(T * k, 2, dtype=torch.int32, device="cuda"),
    )
    try:
        for i, data in enumerate((first, second)):  # two calls in a row on the shared scratch array
            ref, got, moved = _run_both(lib, layer, cfg, data, out)
            _assert_same(cfg, ref, got)
            # the property the entry point exists for: the device's free memory does not move
            # across a call (the very first one may pay for the lazy loading of the kernel image)
            assert i == 0 or moved == 0
    finally:
        layer.close()


def test_noalloc_dispatch_empty_batch_and_bad_expert_id():
    lib = _lib()
    E, k, H, T = 16, 2, 256, 8
    cfg, data, _, _ = contract.make_moe_inputs(E, k, H, T, 5, 0, 1, device="cuda", fixed_num_tokens=T)
    ex = torch.zeros(E, T, H, dtype=cfg.in_dtype, device="cuda")
    em = torch.zeros(E, T, 5, dtype=torch.int32, device="cuda")
    en = torch.full((E,), -1, dtype=torch.int32, device="cuda")
    route = torch.zeros(T * k, 2, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(idx, n_tok):
        return lib.b200_moe_dispatch_noalloc(data.x.data_ptr(), idx.data_ptr(), n_tok, k, H * data.x.element_size(), E, T,
                                             ex.data_ptr(), em.data_ptr(), en.data_ptr(), route.data_ptr(), stream)

    idx = data.indices.to(torch.int32).contiguous()
    assert call(idx, 0) == 0  # no tokens: every expert ends up empty
    assert lib.b200_moe_dispatch_noalloc_status() == 0
    assert en.tolist() == [0] * E
    assert lib.b200_moe_dispatch_noalloc(data.x.data_ptr(), idx.data_ptr(), T, k, H * 2, E, T, None, em.data_ptr(),
                                         en.data_ptr(), route.data_ptr(), stream) == -5  # a null output buffer
    bad = idx.clone()
    bad[3, 1] = E  # one past the last expert
    assert call(bad, T) == 0
    assert lib.b200_moe_dispatch_noalloc_status() == 2  # reported, not faulted
    assert route[3 * k + 1].tolist() == [-1, -1]
    good = [i for i in range(T * k) if i != 3 * k + 1]
    rows = route[good, 1].tolist()
    flat = bad.reshape(-1).tolist()
    for i, row in zip(good, rows):  # every other entry was delivered to its expert
        assert row // T == flat[i] and torch.equal(ex.reshape(E * T, H)[row], data.x[i // k])
    assert int(en.sum()) == T * k - 1
    assert call(idx, T) == 0 and lib.b200_moe_dispatch_noalloc_status() == 0  # the next call starts clean


def test_noalloc_dispatch_rejects_sizes_beyond_its_scratch():
    lib = _lib()
    buf = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = buf.data_ptr()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.b200_moe_dispatch_noalloc(p, p, 4, 2, 64, 4096, 8, p, p, p, p, stream) == -2
    assert b"num_experts" in lib.b200_moe_dispatch_noalloc_error()
    assert lib.b200_moe_dispatch_noalloc(p, p, 40000, 2, 64, 8, 8, p, p, p, p, stream) == -3
    assert b"65536" in lib.b200_moe_dispatch_noalloc_error()
