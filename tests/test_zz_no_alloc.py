"""GPU: the workspace-free Q4_K matmul entry point against the ordinary one.

Some hosts of this library cannot give it device memory: a plugin that is only handed input and
output pointers, or a server that closes its memory pool after start-up.  For them
ub_qmatmul_q4k_f32_static keeps its scratch in a fixed array inside the library.  This file checks,
through the C-ABI, that it returns what ub_qmatmul_q4k_f32 returns with a caller workspace, on two
calls in a row (the second must not see anything left over from the first), and that it refuses
shapes beyond its fixed limit.  It sorts last so that a stop-at-first-failure run has already
executed every other test.
"""
import ctypes

import numpy as np
import pytest

import ubridge_b200 as ub
from oracle import oracle as o
from ubridge_b200 import DTYPE_F32, ops
from ubridge_b200._lib import UB_ERR_TOO_LARGE

pytestmark = pytest.mark.gpu


def _both_ways(dev, seed, M, N, K):
    rng = np.random.default_rng(seed)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, False)
    d_w, d_x = dev.htod_sync_copy(w), dev.htod_sync_copy(x)
    d_ref, d_new = dev.alloc(M * N * 4), dev.alloc(M * N * 4)
    ws_bytes = ops.qmatmul_workspace_bytes(M, N, K, True)
    ws = dev.alloc(max(ws_bytes, 256))
    ops.qmatmul(d_ref, d_x, d_w, M, N, K, is_q4k=True, x_dtype=DTYPE_F32, out_dtype=DTYPE_F32, workspace=ws,
                ws_bytes=ws_bytes, stream=dev.stream)
    ops.qmatmul_q4k_f32_static(d_new, d_x, d_w, M, N, K, DTYPE_F32, stream=dev.stream)
    ref = dev.dtoh_sync_copy(d_ref, np.float32, (M, N))
    new = dev.dtoh_sync_copy(d_new, np.float32, (M, N))
    return ref, new, o.c_qmatmul(x, w, N, K, True)


def test_static_scratch_entry_matches_workspace_entry_twice(dev):
    # two calls in a row with different shapes and data; both use the conversion scratch (M > 16)
    for seed, (M, N, K) in ((1, (40, 264, 1024)), (2, (33, 136, 512))):
        ref, new, exact = _both_ways(dev, seed, M, N, K)
        assert o.rel_l2(new, ref) <= 1e-2          # the tolerance of the tensor-core matmul tests
        assert np.array_equal(new, ref)            # same kernels underneath: identical bits
        assert o.rel_l2(new, exact) <= 1e-2
    # a decode shape needs no scratch at all and still works through this entry
    ref, new, exact = _both_ways(dev, 3, 2, 96, 768)
    assert np.array_equal(new, ref) and o.rel_l2(new, exact) <= 1e-3


def test_static_scratch_entry_rejects_oversized_shapes(dev):
    one = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    st = ub.lib().ub_qmatmul_q4k_f32_static(one, one, one, 2048, 14336, 4096, DTYPE_F32, None)
    assert st == UB_ERR_TOO_LARGE
    assert "limit" in ub.status_string(st)
