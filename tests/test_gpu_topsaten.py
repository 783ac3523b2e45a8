"""GPU parity of the four status-returning `topsaten_*` exports (src/ffi.rs:671-713), called through the C-ABI
with sizes that are all different (tokens != top-k != experts != block), so that a permuted int32 argument
cannot go unnoticed."""
import ctypes

import numpy as np
import pytest

import ubridge_b200 as ub
from oracle import oracle as o
from ubridge_b200 import DTYPE_BF16, DTYPE_F16

from _util import fetch, from_storage, to_storage

pytestmark = pytest.mark.gpu


def _p(buf):
    return ctypes.c_void_p(buf.ptr) if buf is not None else None


def test_topsaten_topk_softmax_f32(dev):
    T, E, k = 37, 12, 3
    rng = np.random.default_rng(11)
    lg = rng.standard_normal((T, E)).astype(np.float32)
    for norm in (0, 1):
        want_w, want_i = o.topk_softmax(lg, k, bool(norm), o.UB_F32)
        d_l, d_w, d_i, d_s = dev.htod_sync_copy(lg), dev.alloc(T * k * 4), dev.alloc(T * k * 4), dev.alloc(T * k * 4)
        st = ub.lib().topsaten_topk_softmax_f32(_p(d_l), _p(d_w), _p(d_i), _p(d_s), T, E, k, norm, dev.stream)
        assert st == 0
        assert np.array_equal(dev.dtoh_sync_copy(d_i, np.int32, (T, k)), want_i)
        assert np.allclose(dev.dtoh_sync_copy(d_w, np.float32, (T, k)), want_w, rtol=1e-6)
        # token_expert_indices: slot (t, j) -> j * T + t
        src = dev.dtoh_sync_copy(d_s, np.int32, (T, k))
        assert np.array_equal(src, np.arange(k)[None, :] * T + np.arange(T)[:, None])
    # NULL token_expert_indices is accepted
    assert ub.lib().topsaten_topk_softmax_f32(_p(d_l), _p(d_w), _p(d_i), None, T, E, k, 0, dev.stream) == 0
    dev.synchronize()


@pytest.mark.parametrize("T,k,E,block", [(37, 3, 12, 5), (256, 2, 8, 64), (5, 4, 9, 16)])
def test_topsaten_moe_align_block_size(dev, T, k, E, block):
    rng = np.random.default_rng(T + E)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    want_s, want_e, want_n = o.c_moe_align(ids, E, block)
    n_sorted = T * k + E * (block - 1)
    n_blocks = n_sorted // block
    d_ids = dev.htod_sync_copy(ids)
    d_s, d_e, d_n = dev.alloc(n_sorted * 4), dev.alloc(max(n_blocks, 1) * 4), dev.alloc(4)
    st = ub.lib().topsaten_moe_align_block_size(_p(d_s), _p(d_e), _p(d_n), _p(d_ids), T, k, E, block, dev.stream)
    assert st == 0
    assert int(dev.dtoh_sync_copy(d_n, np.int32)[0]) == want_n
    assert np.array_equal(dev.dtoh_sync_copy(d_s, np.int32)[:n_sorted], want_s)
    assert np.array_equal(dev.dtoh_sync_copy(d_e, np.int32)[:n_blocks], want_e)


@pytest.mark.parametrize("dtype", [DTYPE_F16, DTYPE_BF16])
@pytest.mark.parametrize("mul", [0, 1])
def test_topsaten_fused_moe_gemm(dev, dtype, mul):
    T, k, E, block, hidden, inter = 21, 3, 5, 8, 64, 40
    rng = np.random.default_rng(5 + mul)
    rows_a = T * k if mul else T
    A = from_storage(to_storage(rng.standard_normal((rows_a, hidden)).astype(np.float32), dtype), dtype)
    B = from_storage(to_storage((rng.standard_normal((E, inter, hidden)) * 0.2).astype(np.float32), dtype), dtype)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    w = rng.uniform(0.1, 1, size=(T, k)).astype(np.float32)
    s, e, npp = o.c_moe_align(ids, E, block)
    odt = o.UB_F16 if dtype == DTYPE_F16 else o.UB_BF16
    want = o.fused_moe(A, B, w, s, e, npp, k, block, mul, odt, T * k)
    d = [dev.htod_sync_copy(v) for v in (to_storage(A, dtype), to_storage(B, dtype), w, ids, s, e,
                                         np.array([npp], dtype=np.int32))]
    d_C = dev.alloc_zeros(T * k * inter * 2)
    st = ub.lib().topsaten_fused_moe_gemm(_p(d_C), _p(d[0]), _p(d[1]), _p(d[2]), _p(d[3]), _p(d[4]), _p(d[5]),
                                          _p(d[6]), mul, k, block, T, hidden, inter, E, dtype, dev.stream)
    assert st == 0
    got = fetch(dev, d_C, dtype, (T * k, inter))
    assert o.rel_l2(got, want) < 2e-3


def test_topsaten_release_graph_workspace_pool_is_a_no_op(dev):
    ub.lib().topsaten_release_graph_workspace_pool(dev.stream)
    dev.synchronize()
    assert dev.device_status() == 0
