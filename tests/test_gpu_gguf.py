"""GPU parity of the GGUF tensor-blob entries: dispatch on the GGML type tag, Q4_0 and Q5_K dequantisation
(bit-exact against the gguf-py-pinned oracle) and their matmul, and the forwarding of the other tags."""
import os

import numpy as np
import pytest

from oracle import oracle as o
from ubridge_b200 import DTYPE_BF16, DTYPE_F16, DTYPE_F32, ops
from ubridge_b200._lib import UB_ERR_UNSUPPORTED, UbridgeError, lib

from _util import ESIZE, fetch, to_storage

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ODT = {DTYPE_F32: o.UB_F32, DTYPE_F16: o.UB_F16, DTYPE_BF16: o.UB_BF16}
GEN = {o.GGML_Q4_0: o.gen_q4_0_weight, o.GGML_Q8_0: o.gen_q8_0_weight, o.GGML_Q4_K: o.gen_q4k_weight,
       o.GGML_Q5_K: o.gen_q5k_weight, o.GGML_Q6_K: o.gen_q6k_weight}
PER = {o.GGML_Q4_0: 32, o.GGML_Q8_0: 32, o.GGML_Q4_K: 256, o.GGML_Q5_K: 256, o.GGML_Q6_K: 256}


def test_golden_blocks_of_the_two_new_formats(dev):
    more = dict(np.load(os.path.join(ROOT, "tests", "golden", "blocks_more.npz")))
    for key, tag in (("q4_0", o.GGML_Q4_0), ("q5k", o.GGML_Q5_K)):
        blob = more[key].reshape(-1)
        want = more[key + "_f32"]
        d_out = dev.alloc(want.size * 4)
        ops.dequantize_gguf(d_out, dev.htod_sync_copy(blob), tag, want.size, DTYPE_F32, stream=dev.stream)
        got = dev.dtoh_sync_copy(d_out, np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), key


@pytest.mark.parametrize("tag", sorted(GEN))
@pytest.mark.parametrize("dtype", [DTYPE_F32, DTYPE_F16, DTYPE_BF16])
def test_dequant_by_type_tag(dev, tag, dtype):
    rng = np.random.default_rng(tag)
    N, K = 37, 1024
    blob = np.ascontiguousarray(GEN[tag](rng, N, K)).reshape(-1)
    assert lib().ub_gguf_tensor_bytes(tag, N * K) == blob.nbytes
    want = o.round_through(o.dequant_gguf(blob, tag), ODT[dtype])
    d_out = dev.alloc(N * K * ESIZE[dtype])
    ops.dequantize_gguf(d_out, dev.htod_sync_copy(blob), tag, N * K, dtype, stream=dev.stream)
    got = fetch(dev, d_out, dtype, (N * K,))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("tag", sorted(GEN))
@pytest.mark.parametrize("x_dtype", [DTYPE_F32, DTYPE_BF16])
@pytest.mark.parametrize("M,N,K", [(1, 130, 1024), (5, 64, 2048), (11, 33, 512)])
def test_matmul_by_type_tag(dev, tag, x_dtype, M, N, K):
    rng = np.random.default_rng(tag * 100 + M)
    blob = np.ascontiguousarray(GEN[tag](rng, N, K)).reshape(-1)
    x = o.gen_activation(rng, M, K, x_dtype == DTYPE_BF16)
    want = o.qmatmul_exact(x, o.dequant_gguf(blob, tag).reshape(N, K))
    ws_bytes = lib().ub_qmatmul_gguf_workspace_bytes(tag, M, N, K)
    ws = dev.alloc(max(ws_bytes, 256))
    d_y = dev.alloc(M * N * 4)
    ops.qmatmul_gguf(d_y, dev.htod_sync_copy(to_storage(x, x_dtype)), dev.htod_sync_copy(blob), tag, M, N, K,
                     x_dtype=x_dtype, out_dtype=DTYPE_F32, workspace=ws, ws_bytes=ws_bytes, stream=dev.stream)
    got = dev.dtoh_sync_copy(d_y, np.float32, (M, N))
    assert o.rel_l2(got, want) < 1e-3


@pytest.mark.parametrize("x_dtype,out_dtype", [(DTYPE_BF16, DTYPE_F32), (DTYPE_F32, DTYPE_F32), (DTYPE_BF16, DTYPE_BF16)])
@pytest.mark.parametrize("M,N,K", [(1, 1, 4096), (1, 9, 2048), (1, 4747, 4096), (1, 30000, 4096), (1, 3001, 8192),
                                   (1, 1000, 14336), (2, 2369, 2048), (3, 4747, 4096), (4, 14336, 4096), (7, 1000, 4096),
                                   (4, 300, 14336)])
def test_q5k_rows_staged_by_bulk_copies(dev, x_dtype, out_dtype, M, N, K):
    """Q5_K with rows of whole 2048 values, one to four tokens per pass: rows staged by bulk copies, 15-bit
    fixed-point activations.  Fewer rows than CTAs, row ranges of unequal length, more stages per CTA than the ring
    has slots (30000 rows), a last stage of fewer than eight rows, one CTA per SM for long rows, the fall-back when
    four tokens of 14336 values do not fit."""
    tag = o.GGML_Q5_K
    rng = np.random.default_rng(M + N + K)
    blob = np.ascontiguousarray(o.gen_q5k_weight(rng, N, K)).reshape(-1)
    x = o.gen_activation(rng, M, K, x_dtype == DTYPE_BF16)
    x[M - 1] *= 512.0  # every token has its own scales
    want = o.qmatmul_exact(x, o.dequant_gguf(blob, tag).reshape(N, K))
    d_w, d_x = dev.htod_sync_copy(blob), dev.htod_sync_copy(to_storage(x, x_dtype))

    def run(dt):
        d_y = dev.alloc(M * N * ESIZE[dt])
        ops.qmatmul_gguf(d_y, d_x, d_w, tag, M, N, K, x_dtype=x_dtype, out_dtype=dt, stream=dev.stream)
        return fetch(dev, d_y, dt, (M, N))

    got = run(DTYPE_F32)
    for m in range(M):
        assert o.rel_l2(got[m], want[m]) < (1e-4 if N >= 1000 else 1e-3), m
    assert np.array_equal(got, run(DTYPE_F32))  # fixed summation order
    if out_dtype != DTYPE_F32:
        assert np.array_equal(run(out_dtype), o.round_through(got, ODT[out_dtype]))


@pytest.mark.parametrize("x_dtype,out_dtype", [(DTYPE_BF16, DTYPE_F32), (DTYPE_F32, DTYPE_F32), (DTYPE_BF16, DTYPE_BF16)])
@pytest.mark.parametrize("M,N,K", [(1, 1, 4096), (1, 9, 2048), (1, 4747, 4096), (1, 30000, 4096), (1, 3001, 8192),
                                   (1, 1000, 14336), (2, 2369, 2048), (3, 4747, 4096), (4, 14336, 4096), (7, 1000, 4096),
                                   (4, 300, 28672)])
def test_q4_0_rows_staged_by_bulk_copies(dev, x_dtype, out_dtype, M, N, K):
    """Q4_0 with rows of whole 2048 values, one to four tokens per pass: the same cases as for Q5_K; blocks of 18
    bytes alternate between a 4-byte boundary and two bytes past one."""
    tag = o.GGML_Q4_0
    rng = np.random.default_rng(M + N + K)
    blob = np.ascontiguousarray(o.gen_q4_0_weight(rng, N, K)).reshape(-1)
    x = o.gen_activation(rng, M, K, x_dtype == DTYPE_BF16)
    x[M - 1] *= 512.0  # every token has its own scales
    x[0, 256:512] = 0.0
    want = o.qmatmul_exact(x, o.dequant_gguf(blob, tag).reshape(N, K))
    d_w, d_x = dev.htod_sync_copy(blob), dev.htod_sync_copy(to_storage(x, x_dtype))

    def run(dt):
        d_y = dev.alloc(M * N * ESIZE[dt])
        ops.qmatmul_gguf(d_y, d_x, d_w, tag, M, N, K, x_dtype=x_dtype, out_dtype=dt, stream=dev.stream)
        return fetch(dev, d_y, dt, (M, N))

    got = run(DTYPE_F32)
    for m in range(M):
        assert o.rel_l2(got[m], want[m]) < (1e-4 if N >= 1000 else 1e-3), m
    assert np.array_equal(got, run(DTYPE_F32))  # fixed summation order
    if out_dtype != DTYPE_F32:
        assert np.array_equal(run(out_dtype), o.round_through(got, ODT[out_dtype]))


def test_q4_0_staged_extreme_blocks(dev):
    """Every nibble pattern (rows of all 0 and all 15 among them), negative and tiny scales."""
    tag = o.GGML_Q4_0
    rng = np.random.default_rng(40)
    N, K = 520, 4096
    raw = rng.integers(0, 256, size=(N, K // 32, 18), dtype=np.uint8)
    raw[:, :, 0:2] = rng.uniform(-0.05, 0.05, size=(N, K // 32)).astype(np.float16).view(np.uint8).reshape(N, K // 32, 2)
    raw[0, :, 2:] = 0xFF
    raw[1, :, 2:] = 0x00
    blob = raw.reshape(-1)
    x = o.gen_activation(rng, 1, K, True)
    want = o.qmatmul_exact(x, o.dequant_gguf(blob, tag).reshape(N, K))
    d_y = dev.alloc(N * 4)
    ops.qmatmul_gguf(d_y, dev.htod_sync_copy(to_storage(x, DTYPE_BF16)), dev.htod_sync_copy(blob), tag, 1, N, K,
                     x_dtype=DTYPE_BF16, out_dtype=DTYPE_F32, stream=dev.stream)
    got = fetch(dev, d_y, DTYPE_F32, (1, N))
    assert o.rel_l2(got, want) < 1e-4
    assert np.allclose(got[0, :2], want[0, :2], rtol=2e-4, atol=1e-3 * np.abs(want).max())


def test_q5k_staged_extreme_blocks(dev):
    """Every bit pattern of the nibbles, the fifth bits and the 6-bit scales and mins; zero and large activations."""
    tag = o.GGML_Q5_K
    rng = np.random.default_rng(55)
    N, K = 520, 4096
    raw = rng.integers(0, 256, size=(N, K // 256, 176), dtype=np.uint8)
    raw[:, :, 0:2] = rng.uniform(1e-4, 1e-2, size=(N, K // 256)).astype(np.float16).view(np.uint8).reshape(N, K // 256, 2)
    raw[:, :, 2:4] = rng.uniform(1e-4, 1e-2, size=(N, K // 256)).astype(np.float16).view(np.uint8).reshape(N, K // 256, 2)
    raw[0, :, 4:] = 0xFF  # q = 31, scales and mins 63 everywhere
    raw[1, :, 4:] = 0x00
    blob = raw.reshape(-1)
    x = o.gen_activation(rng, 1, K, True)
    x[0, :256] = 0.0
    x[0, 256:512] *= 8192.0
    want = o.qmatmul_exact(x, o.dequant_gguf(blob, tag).reshape(N, K))
    d_y = dev.alloc(N * 4)
    ops.qmatmul_gguf(d_y, dev.htod_sync_copy(to_storage(x, DTYPE_BF16)), dev.htod_sync_copy(blob), tag, 1, N, K,
                     x_dtype=DTYPE_BF16, out_dtype=DTYPE_F32, stream=dev.stream)
    got = fetch(dev, d_y, DTYPE_F32, (1, N))
    assert o.rel_l2(got, want) < 1e-4
    assert np.allclose(got[0, :2], want[0, :2], rtol=2e-4, atol=1e-3 * np.abs(want).max())


def test_unknown_type_tag_is_refused(dev):
    d = dev.alloc(4096)
    with pytest.raises(UbridgeError) as ei:
        ops.dequantize_gguf(d, d, 10, 256, DTYPE_F32, stream=dev.stream)  # Q2_K: declared upstream, not taken here
    assert ei.value.status == UB_ERR_UNSUPPORTED
    assert lib().ub_gguf_tensor_bytes(10, 256) == 0
