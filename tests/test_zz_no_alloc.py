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
from ubridge_b200 import DTYPE_BF16, DTYPE_F16, DTYPE_F32, ops
from ubridge_b200._lib import UB_ERR_TOO_LARGE

pytestmark = pytest.mark.gpu


_NP_OF = {DTYPE_F32: np.float32, DTYPE_F16: np.float16, DTYPE_BF16: np.uint16}


def _to_f32(a, dtype):
    return o.bf16_bits_to_f32(a) if dtype == DTYPE_BF16 else a.astype(np.float32)


def _both_ways(dev, seed, M, N, K, out_dtype=DTYPE_F32):
    rng = np.random.default_rng(seed)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, False)
    d_w, d_x = dev.htod_sync_copy(w), dev.htod_sync_copy(x)
    d_ref, d_new = dev.alloc(M * N * 4), dev.alloc(M * N * 4)
    ws_bytes = ops.qmatmul_workspace_bytes(M, N, K, True)
    ws = dev.alloc(max(ws_bytes, 256))
    ops.qmatmul(d_ref, d_x, d_w, M, N, K, is_q4k=True, x_dtype=DTYPE_F32, out_dtype=out_dtype, workspace=ws,
                ws_bytes=ws_bytes, stream=dev.stream)
    ops.qmatmul_q4k_f32_static(d_new, d_x, d_w, M, N, K, out_dtype, stream=dev.stream)
    npdt = _NP_OF[out_dtype]
    ref = dev.dtoh_sync_copy(d_ref, npdt)[: M * N].reshape(M, N)
    new = dev.dtoh_sync_copy(d_new, npdt)[: M * N].reshape(M, N)
    return _to_f32(ref, out_dtype), _to_f32(new, out_dtype), o.c_qmatmul(x, w, N, K, True)


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


@pytest.mark.parametrize("out_dtype", [DTYPE_BF16, DTYPE_F16])
def test_static_scratch_entry_other_output_types(dev, out_dtype):
    # bf16 output needs only the activation half of the scratch, f16 output both halves
    for seed, (M, N, K) in ((4, (40, 264, 1024)), (5, (17, 128, 256))):
        ref, new, exact = _both_ways(dev, seed, M, N, K, out_dtype)
        assert np.array_equal(new, ref)
        assert o.rel_l2(new, exact) <= 1e-2


def test_static_scratch_entry_at_its_limit(dev):
    # M (K + N) = 4 Mi elements: the scratch need is exactly the 8 MiB of the fixed array
    M, N, K = 1024, 2048, 2048
    assert ops.qmatmul_workspace_bytes(M, N, K, True) == 8 << 20
    ref, new, exact = _both_ways(dev, 6, M, N, K)
    assert np.array_equal(new, ref) and o.rel_l2(new, exact) <= 1e-2
    # 256 bytes more (one more output column at 128 tokens) is refused before anything is touched
    assert ops.qmatmul_workspace_bytes(128, 16384, 16384, True) == 8 << 20
    assert ops.qmatmul_workspace_bytes(128, 16385, 16384, True) == (8 << 20) + 256
    one = ctypes.c_void_p(256)
    assert ub.lib().ub_qmatmul_q4k_f32_static(one, one, one, 128, 16385, 16384, DTYPE_F32, None) == UB_ERR_TOO_LARGE


def test_static_scratch_entry_leaves_free_memory_unchanged(dev):
    """The property in the entry point's name: after a first call (which may load code lazily), further calls
    change nothing in the device's free memory."""
    rng = np.random.default_rng(7)
    M, N, K = 64, 512, 1024
    w, x = o.gen_q4k_weight(rng, N, K), o.gen_activation(rng, M, K, False)
    d_w, d_x, d_y = dev.htod_sync_copy(w), dev.htod_sync_copy(x), dev.alloc(M * N * 4)
    ops.qmatmul_q4k_f32_static(d_y, d_x, d_w, M, N, K, DTYPE_F32, stream=dev.stream)
    dev.synchronize()
    free0, _total = dev.mem_info()
    for _ in range(3):
        ops.qmatmul_q4k_f32_static(d_y, d_x, d_w, M, N, K, DTYPE_F32, stream=dev.stream)
    dev.synchronize()
    free1, _total = dev.mem_info()
    assert free1 == free0
