"""GPU parity: GGUF Q6_K dequantisation (bit-exact) and the Q6_K decode matmul (rel-L2 <= 1e-3, f32
accumulation) through the C-ABI, against the oracle and the known-answer fixtures."""
import numpy as np
import pytest

from oracle import oracle as o
from ubridge_b200 import DTYPE_BF16, DTYPE_F16, DTYPE_F32, UbridgeError, ops
from ubridge_b200._lib import UB_ERR_INVALID_ARG

from _util import ESIZE, fetch, to_storage

pytestmark = pytest.mark.gpu

TOL_DECODE = 1e-3


def _expect(values_f32, dtype):
    return o.round_through(values_f32, {DTYPE_F32: o.UB_F32, DTYPE_F16: o.UB_F16, DTYPE_BF16: o.UB_BF16}[dtype])


def _dequant(dev, blocks, dtype):
    n = blocks.size // o.Q6K_BYTES * o.QK_K
    d_in = dev.htod_sync_copy(np.ascontiguousarray(blocks).reshape(-1))
    d_out = dev.alloc(n * ESIZE[dtype])
    ops.dequantize_q6k(d_out, d_in, n, dtype, stream=dev.stream)
    return fetch(dev, d_out, dtype, (n,))


def _matmul(dev, w, x, M, N, K, x_dtype, out_dtype):
    d_w = dev.htod_sync_copy(np.ascontiguousarray(w).reshape(-1))
    d_x = dev.htod_sync_copy(to_storage(x, x_dtype))
    d_y = dev.alloc(M * N * ESIZE[out_dtype])
    ops.qmatmul_q6k(d_y, d_x, d_w, M, N, K, x_dtype=x_dtype, out_dtype=out_dtype, stream=dev.stream)
    return fetch(dev, d_y, out_dtype, (M, N))


def test_golden_blocks(dev, golden):
    for key in ("hand_q6k_block", "rand_q6k_blocks"):
        expect = golden[key.replace("_blocks", "_expect").replace("_block", "_expect")].reshape(-1)
        got = _dequant(dev, golden[key], DTYPE_F32)
        assert np.array_equal(got.view(np.uint32), expect.view(np.uint32)), key


@pytest.mark.parametrize("dtype", [DTYPE_F32, DTYPE_F16, DTYPE_BF16])
@pytest.mark.parametrize("nblocks", [1, 7, 1000])
def test_dequant_bit_exact(dev, dtype, nblocks):
    rng = np.random.default_rng(nblocks)
    raw = rng.integers(0, 256, size=(nblocks, o.Q6K_BYTES), dtype=np.uint8)  # every bit pattern of ql, qh, scales
    raw[:, 208:210] = rng.uniform(-0.05, 0.05, size=nblocks).astype(np.float16).view(np.uint8).reshape(nblocks, 2)
    got = _dequant(dev, raw, dtype)
    want = _expect(o.dequant_q6k(raw).reshape(-1), dtype)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_full_size_weight_and_empty_input(dev):
    """A 14336 x 4096 matrix (48 MB of blocks) and numel = 0."""
    rng = np.random.default_rng(1006)
    w = o.gen_q6k_weight(rng, 14336, 4096)
    got = _dequant(dev, w, DTYPE_BF16)
    want = _expect(o.dequant_q6k(w).reshape(-1), DTYPE_BF16)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    ops.dequantize_q6k(None, None, 0, DTYPE_F32, stream=dev.stream)  # nothing to do, no error
    with pytest.raises(UbridgeError) as ei:
        ops.dequantize_q6k(dev.alloc(1024), dev.alloc(1024), 100, DTYPE_F32, stream=dev.stream)
    assert ei.value.status == UB_ERR_INVALID_ARG


def test_golden_matmul(dev, golden):
    got = _matmul(dev, golden["mm_q6k_w"], golden["mm_q6k_x"], 5, 24, 512, DTYPE_F32, DTYPE_F32)
    assert o.rel_l2(got, golden["mm_q6k_y"]) < 1e-5


@pytest.mark.parametrize("x_dtype", [DTYPE_F32, DTYPE_BF16])
@pytest.mark.parametrize("M,N,K", [(1, 1, 256), (2, 7, 256), (3, 33, 768), (5, 130, 1024), (9, 257, 2048), (1, 64, 14336)])
def test_matmul_odd_shapes(dev, x_dtype, M, N, K):
    rng = np.random.default_rng(M * 1000 + N)
    w = o.gen_q6k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, x_dtype == DTYPE_BF16)
    want = o.qmatmul_exact(x, o.dequant_q6k(w).reshape(N, K))
    got = _matmul(dev, w, x, M, N, K, x_dtype, DTYPE_F32)
    assert o.rel_l2(got, want) < TOL_DECODE
    if K % 2048:
        assert o.rel_l2(got, want) < 1e-5  # f32 products of exact weights: only the summation order differs
    else:
        assert o.rel_l2(got, want) < 1e-4  # rows of whole 2048 values: 15-bit fixed-point activations


@pytest.mark.parametrize("x_dtype,out_dtype", [(DTYPE_BF16, DTYPE_F32), (DTYPE_F32, DTYPE_F32), (DTYPE_BF16, DTYPE_BF16),
                                               (DTYPE_F32, DTYPE_F16)])
@pytest.mark.parametrize("N,K", [(1, 4096), (9, 2048), (17, 4096), (4747, 4096), (2369, 2048), (30000, 4096), (20000, 2048),
                                 (3001, 8192), (2000, 14336), (700, 6144)])
def test_single_token_staged_kernel(dev, x_dtype, out_dtype, N, K):
    """One token at K a multiple of 2048: rows staged by bulk copies, 15-bit fixed-point activations.  Fewer rows
    than CTAs, row ranges of unequal length, more stages per CTA than the ring has slots (30000 rows), a last stage
    of fewer than eight rows; rows of 6144 to 14336 values run one CTA per SM."""
    rng = np.random.default_rng(N + K)
    w = o.gen_q6k_weight(rng, N, K)
    x = o.gen_activation(rng, 1, K, x_dtype == DTYPE_BF16)
    want = o.qmatmul_exact(x, o.dequant_q6k(w).reshape(N, K))
    got = _matmul(dev, w, x, 1, N, K, x_dtype, out_dtype)
    if out_dtype == DTYPE_F32:
        assert o.rel_l2(got, want) < (1e-4 if N >= 1000 else TOL_DECODE)
        assert np.array_equal(got, _matmul(dev, w, x, 1, N, K, x_dtype, out_dtype))  # fixed summation order
    else:
        assert np.array_equal(got, _expect(_matmul(dev, w, x, 1, N, K, x_dtype, DTYPE_F32), out_dtype))


@pytest.mark.parametrize("M,N,K", [(2, 4747, 4096), (3, 2369, 2048), (4, 14336, 4096), (7, 1000, 4096), (4, 900, 8192),
                                   (2, 300, 14336), (4, 300, 14336)])
def test_two_to_four_tokens_staged_kernel(dev, M, N, K):
    """The staged kernel with two or four token slots (three tokens: the fourth slot is not computed; seven: a pass
    of four and one of three); 14336-value rows fit with two tokens and fall back to the streaming kernel with four."""
    rng = np.random.default_rng(M + N + K)
    w = o.gen_q6k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    x[M - 1] *= 512.0  # every token has its own scales
    want = o.qmatmul_exact(x, o.dequant_q6k(w).reshape(N, K))
    got = _matmul(dev, w, x, M, N, K, DTYPE_BF16, DTYPE_F32)
    for m in range(M):
        assert o.rel_l2(got[m], want[m]) < 1e-4, m
    assert np.array_equal(got, _matmul(dev, w, x, M, N, K, DTYPE_BF16, DTYPE_F32))
    got16 = _matmul(dev, w, x, M, N, K, DTYPE_BF16, DTYPE_BF16)
    assert np.array_equal(got16, _expect(got, DTYPE_BF16))


def test_single_token_staged_kernel_extreme_blocks(dev):
    """Every bit pattern of ql, qh and the int8 scales (among them -128 and 127), zero and large activations."""
    rng = np.random.default_rng(66)
    N, K = 520, 4096
    raw = rng.integers(0, 256, size=(N, K // 256, o.Q6K_BYTES), dtype=np.uint8)
    raw[:, :, 208:210] = rng.uniform(-0.05, 0.05, size=(N, K // 256)).astype(np.float16).view(np.uint8).reshape(N, K // 256, 2)
    raw[0, 0, 192:208] = 0x80  # scales of -128
    raw[1, 0, 192:208] = 0x7F
    raw[2, :, :192] = 0xFF     # q = 63 everywhere
    raw[3, :, :192] = 0x00     # q = 0 everywhere
    x = o.gen_activation(rng, 1, K, True)
    x[0, :256] = 0.0
    x[0, 256:512] *= 8192.0
    got = _matmul(dev, raw, x, 1, N, K, DTYPE_BF16, DTYPE_F32)
    want = o.qmatmul_exact(x, o.dequant_q6k(raw).reshape(N, K))
    assert o.rel_l2(got, want) < 1e-4
    assert np.allclose(got[0, :4], want[0, :4], rtol=2e-4, atol=1e-3 * np.abs(want).max())


def test_matmul_weights_on_a_two_byte_boundary(dev):
    """GGUF tensors inside a mapped file need not start on a 4-byte boundary: the kernel's 16-bit-load path."""
    rng = np.random.default_rng(21)
    M, N, K = 2, 40, 1792
    w = o.gen_q6k_weight(rng, N, K).reshape(-1)
    x = o.gen_activation(rng, M, K, True)
    buf = dev.alloc(w.size + 16)
    d_w = buf.slice(2, 2 + w.size)
    dev.htod_copy_into(w, d_w)
    d_x = dev.htod_sync_copy(to_storage(x, DTYPE_BF16))
    d_y = dev.alloc(M * N * 4)
    ops.qmatmul_q6k(d_y, d_x, d_w, M, N, K, x_dtype=DTYPE_BF16, out_dtype=DTYPE_F32, stream=dev.stream)
    got = fetch(dev, d_y, DTYPE_F32, (M, N))
    aligned = _matmul(dev, w, x, M, N, K, DTYPE_BF16, DTYPE_F32)
    assert np.array_equal(got, aligned)  # same arithmetic, only the loads differ
    assert o.rel_l2(got, o.qmatmul_exact(x, o.dequant_q6k(w.reshape(N, K // 256, 210)).reshape(N, K))) < 1e-5


def test_matmul_full_size_decode(dev):
    """Q6_K 14336 x 4096, bf16 activations, M = 1 and 4, bf16 and f32 output; doubling x doubles y exactly."""
    rng = np.random.default_rng(1006)
    N, K = 14336, 4096
    w = o.gen_q6k_weight(rng, N, K)
    wd = o.dequant_q6k(w).reshape(N, K)
    for M in (1, 4):
        x = o.gen_activation(rng, M, K, True)
        want = o.qmatmul_exact(x, wd)
        got32 = _matmul(dev, w, x, M, N, K, DTYPE_BF16, DTYPE_F32)
        assert o.rel_l2(got32, want) < TOL_DECODE
        got16 = _matmul(dev, w, x, M, N, K, DTYPE_BF16, DTYPE_BF16)
        assert np.array_equal(got16, o.round_through(got32, o.UB_BF16))
        assert np.array_equal(_matmul(dev, w, 2 * x, M, N, K, DTYPE_BF16, DTYPE_F32), 2 * got32)


def test_matmul_rejects_bad_shapes(dev):
    buf = dev.alloc(4096)
    with pytest.raises(UbridgeError) as ei:
        ops.qmatmul_q6k(buf, buf, buf, 1, 4, 100, x_dtype=DTYPE_F32, out_dtype=DTYPE_F32, stream=dev.stream)
    assert ei.value.status == UB_ERR_INVALID_ARG
    ops.qmatmul_q6k(buf, buf, buf, 0, 4, 256, x_dtype=DTYPE_F32, out_dtype=DTYPE_F32, stream=dev.stream)  # M = 0
