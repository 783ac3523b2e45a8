"""GPU parity: fused dequantise + matmul through the C-ABI against the exact oracle.

Tolerances are the ones the task states: rel-L2 <= 1e-3 for the f32-accumulate decode kernel,
<= 1e-2 for the bf16 tensor-core path (its weights are rounded to bf16 once)."""
import numpy as np
import pytest

from oracle import oracle as o
from ubridge_b200 import DTYPE_BF16, DTYPE_F16, DTYPE_F32, ops
from ubridge_b200._lib import UB_ERR_WORKSPACE, UbridgeError

from _util import ESIZE, fetch, to_storage

pytestmark = pytest.mark.gpu

TOL_DECODE = 1e-3
TOL_TENSOR = 1e-2


def _run(dev, wq, x_f32, M, N, K, is_q4k, x_dtype, out_dtype):
    d_w = dev.htod_sync_copy(wq)
    d_x = dev.htod_sync_copy(to_storage(x_f32, x_dtype))
    d_y = dev.alloc(M * N * ESIZE[out_dtype])
    ws_bytes = ops.qmatmul_workspace_bytes(M, N, K, is_q4k)
    ws = dev.alloc(max(ws_bytes, 256))
    ops.qmatmul(d_y, d_x, d_w, M, N, K, is_q4k=is_q4k, x_dtype=x_dtype, out_dtype=out_dtype, workspace=ws,
                ws_bytes=ws_bytes, stream=dev.stream)
    return fetch(dev, d_y, out_dtype, (M, N))


def test_golden_matmuls(dev, golden):
    for name, is_q4k, N, K in (("mm_q8_0", False, 24, 256), ("mm_q4k", True, 24, 512)):
        w, x, y = golden[name + "_w"], golden[name + "_x"], golden[name + "_y"]
        got = _run(dev, w, x, 5, N, K, is_q4k, DTYPE_F32, DTYPE_F32)
        assert o.rel_l2(got, y) < 1e-4, name  # f32 accumulation around a biased nibble encoding


def test_config1_q8_0_decode(dev):
    """Q8_0 4096x4096, x f32 1x4096, y f32."""
    rng = np.random.default_rng(1001)
    N = K = 4096
    w = o.gen_q8_0_weight(rng, N, K)
    x = o.gen_activation(rng, 1, K, False)
    got = _run(dev, w, x, 1, N, K, False, DTYPE_F32, DTYPE_F32)
    want = o.c_qmatmul(x, w, N, K, False)
    assert o.rel_l2(got, want) < TOL_DECODE
    # exact integer dots of 15-bit block fixed-point activations (relative step 2^-15): far inside the tolerance
    assert o.rel_l2(got, want) < 1e-4


@pytest.mark.parametrize("M", [1, 4, 16])
def test_config2_q4k_small_batch(dev, M):
    """Q4_K 14336x4096, bf16 activations M in {1,4,16}, bf16 output."""
    rng = np.random.default_rng(1002)
    N, K = 14336, 4096
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    want = o.c_qmatmul(x, w, N, K, True)
    got32 = _run(dev, w, x, M, N, K, True, DTYPE_BF16, DTYPE_F32)
    assert o.rel_l2(got32, want) < TOL_DECODE
    got16 = _run(dev, w, x, M, N, K, True, DTYPE_BF16, DTYPE_BF16)
    if M <= 8:
        assert np.array_equal(got16, o.round_through(got32, o.UB_BF16))  # output rounding is the only difference
        assert o.rel_l2(got16, want) < 4e-3  # bf16 storage of y alone costs ~2e-3
    else:  # bf16 in and out from nine tokens on: the tensor-core kernel (weights rounded to bf16 once)
        assert o.rel_l2(got16, want) < TOL_TENSOR
        assert o.rel_l2(got16, want) < 5e-3


@pytest.mark.parametrize("is_q4k", [False, True])
@pytest.mark.parametrize("x_dtype", [DTYPE_F32, DTYPE_BF16])
@pytest.mark.parametrize("M,N,K", [(1, 1, 256), (2, 7, 256), (3, 33, 768), (5, 130, 1024), (16, 257, 2048), (7, 64, 14336)])
def test_decode_odd_shapes(dev, is_q4k, x_dtype, M, N, K):
    rng = np.random.default_rng(M * 1000 + N)
    w = (o.gen_q4k_weight if is_q4k else o.gen_q8_0_weight)(rng, N, K)
    x = o.gen_activation(rng, M, K, x_dtype == DTYPE_BF16)
    got = _run(dev, w, x, M, N, K, is_q4k, x_dtype, DTYPE_F32)
    assert o.rel_l2(got, o.c_qmatmul(x, w, N, K, is_q4k)) < TOL_DECODE


@pytest.mark.parametrize("M,N,K", [(9, 33, 768), (12, 257, 2048), (16, 130, 1024)])
def test_q4k_bf16_nine_to_sixteen_tokens(dev, M, N, K):
    """bf16 in and out with 9..16 tokens: one tensor-core launch, no workspace; other types keep the decode kernel."""
    rng = np.random.default_rng(M * 1000 + N)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    want = o.c_qmatmul(x, w, N, K, True)
    assert ops.qmatmul_workspace_bytes(M, N, K, True) == 0
    assert o.rel_l2(_run(dev, w, x, M, N, K, True, DTYPE_BF16, DTYPE_BF16), want) < TOL_TENSOR
    assert o.rel_l2(_run(dev, w, x, M, N, K, True, DTYPE_BF16, DTYPE_F32), want) < TOL_DECODE


def test_q8_0_k_not_multiple_of_256(dev):
    rng = np.random.default_rng(77)
    M, N, K = 2, 19, 96
    w = o.gen_q8_0_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, False)
    got = _run(dev, w, x, M, N, K, False, DTYPE_F32, DTYPE_F32)
    assert o.rel_l2(got, o.c_qmatmul(x, w, N, K, False)) < 1e-4


@pytest.mark.parametrize("M", [17, 63, 64, 65, 200])
def test_q4k_general_m(dev, M):
    rng = np.random.default_rng(300 + M)
    N, K = 264, 1024
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    want = o.c_qmatmul(x, w, N, K, True)
    got = _run(dev, w, x, M, N, K, True, DTYPE_BF16, DTYPE_BF16)
    assert o.rel_l2(got, want) < TOL_TENSOR
    got32 = _run(dev, w, x, M, N, K, True, DTYPE_F32, DTYPE_F32)  # converted through the workspace
    assert o.rel_l2(got32, want) < TOL_TENSOR


def _bf16_weights_product(x, w, N, K):
    """x . W^T with the dequantised Q8_0 weights rounded to bf16 first: what the tensor-core kernel multiplies."""
    wd = o.round_through(o.c_dequant(w, False).reshape(N, K), o.UB_BF16)
    return x.astype(np.float64) @ wd.astype(np.float64).T


@pytest.mark.parametrize("is_q4k", [True, False])
@pytest.mark.parametrize("M,N,K", [(5, 4096, 4096), (16, 4096, 4096), (64, 4096, 4096), (33, 8192, 4096), (16, 14336, 4096),
                                   (7, 1000, 2048), (16, 130, 512), (20, 30000, 2048), (48, 20000, 1024),
                                   (9, 300, 8192), (64, 640, 28672)])
def test_few_tokens_k_split(dev, is_q4k, M, N, K):
    """5 to 64 tokens on the tensor-core kernel: tiles split along K over clusters of 2, 4 or 8 CTAs (4096 rows of 4096:
    8; 8192 rows: 4; 14336: 2), partial sums exchanged through the cluster's shared memory; more tiles than clusters
    (30000 and 20000 rows, so the exchange buffers are reused), ragged last tiles, every token count's owner pattern.
    Fixed summation order: two runs agree bit for bit."""
    rng = np.random.default_rng(M + N + K)
    w = o.gen_q4k_weight(rng, N, K) if is_q4k else o.gen_q8_0_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    got = _run(dev, w, x, M, N, K, is_q4k, DTYPE_BF16, DTYPE_BF16)
    want = x @ o.c_dequant(w, is_q4k).reshape(N, K).T
    err = o.rel_l2(got, want)
    # weights and outputs pass through bf16 (2^-9 each): ~3e-3 overall; a misplaced partial sum would show as 0.1-1
    assert err < 5e-3, err
    assert np.array_equal(got, _run(dev, w, x, M, N, K, is_q4k, DTYPE_BF16, DTYPE_BF16))


@pytest.mark.parametrize("M", [17, 64, 65, 130, 300])
def test_q8_0_general_m(dev, M):
    """Q8_0 with more than 16 tokens: the tcgen05 kernel with the Q8_0 producer (K % 256 == 0, aligned weights)."""
    rng = np.random.default_rng(400 + M)
    N, K = 264, 1024
    w = o.gen_q8_0_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    want = o.c_qmatmul(x, w, N, K, False)
    got = _run(dev, w, x, M, N, K, False, DTYPE_BF16, DTYPE_BF16)
    assert o.rel_l2(got, want) < TOL_TENSOR
    # the only differences from the exact product: weights rounded to bf16 once, output rounded to bf16 once
    assert o.rel_l2(got, _bf16_weights_product(x, w, N, K)) < 3e-3
    got32 = _run(dev, w, x, M, N, K, False, DTYPE_F32, DTYPE_F16)  # converted through the workspace
    assert o.rel_l2(got32, want) < TOL_TENSOR


def test_q8_0_general_m_without_tensor_core_preconditions(dev):
    """Rows that are not whole 16-byte pieces, or no workspace for the conversions: the decode kernel in passes."""
    rng = np.random.default_rng(401)
    M, N, K = 40, 96, 288
    w = o.gen_q8_0_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    got = _run(dev, w, x, M, N, K, False, DTYPE_BF16, DTYPE_F32)
    assert o.rel_l2(got, o.c_qmatmul(x, w, N, K, False)) < TOL_DECODE
    M, N, K = 40, 96, 512
    w = o.gen_q8_0_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, False)
    d_w, d_x, d_y = dev.htod_sync_copy(w), dev.htod_sync_copy(x), dev.alloc(M * N * 4)
    ops.qmatmul(d_y, d_x, d_w, M, N, K, is_q4k=False, x_dtype=DTYPE_F32, out_dtype=DTYPE_F32, stream=dev.stream)
    assert o.rel_l2(fetch(dev, d_y, DTYPE_F32, (M, N)), o.c_qmatmul(x, w, N, K, False)) < TOL_DECODE


def test_q8_0_prefill_full_size(dev):
    """Q8_0 4096x4096 (the C1 weight) with 512 bf16 tokens."""
    rng = np.random.default_rng(1001)
    N = K = 4096
    M = 512
    w = o.gen_q8_0_weight(rng, N, K)
    x = o.gen_activation(np.random.default_rng(1003), M, K, True)
    got = _run(dev, w, x, M, N, K, False, DTYPE_BF16, DTYPE_BF16)
    want = x @ o.c_dequant(w, False).reshape(N, K).T
    assert o.rel_l2(got, want) < TOL_TENSOR
    assert o.rel_l2(got, want) < 3e-3
    # linearity: doubling the activations doubles every output exactly (powers of two commute with rounding)
    got1 = _run(dev, w, x[:64], 64, N, K, False, DTYPE_BF16, DTYPE_BF16)
    got2 = _run(dev, w, 2 * x[:64], 64, N, K, False, DTYPE_BF16, DTYPE_BF16)
    assert np.array_equal(got2, 2 * got1)
    assert o.rel_l2(got1, got[:64]) < 1e-3  # 64 tokens split K over several CTAs: another summation order


def test_workspace_is_required_when_types_need_conversion(dev):
    rng = np.random.default_rng(1)
    M, N, K = 64, 64, 256
    d_w = dev.htod_sync_copy(o.gen_q4k_weight(rng, N, K))
    d_x = dev.htod_sync_copy(o.gen_activation(rng, M, K, False))
    d_y = dev.alloc(M * N * 4)
    with pytest.raises(UbridgeError) as ei:
        ops.qmatmul(d_y, d_x, d_w, M, N, K, is_q4k=True, x_dtype=DTYPE_F32, out_dtype=DTYPE_F32, stream=dev.stream)
    assert ei.value.status == UB_ERR_WORKSPACE


def test_config3_q4k_prefill_full_size(dev):
    """Q4_K 14336x4096 with bf16 activations 2048x4096 -> bf16 2048x14336 (f32 accumulate)."""
    rng = np.random.default_rng(1002)
    N, K, M = 14336, 4096, 2048
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(np.random.default_rng(1003), M, K, True)
    got = _run(dev, w, x, M, N, K, True, DTYPE_BF16, DTYPE_BF16)
    wd = o.c_dequant(w, True).reshape(N, K)
    want = x @ wd.T  # f32 BLAS on the host: the full-size check is against 1e-2, not bit-exactness
    assert o.rel_l2(got, want) < TOL_TENSOR
    # linearity: doubling the activations doubles every output exactly (powers of two commute with rounding)
    got1 = _run(dev, w, x[:64], 64, N, K, True, DTYPE_BF16, DTYPE_BF16)
    got2 = _run(dev, w, 2 * x[:64], 64, N, K, True, DTYPE_BF16, DTYPE_BF16)
    assert np.array_equal(got2, 2 * got1)
    assert o.rel_l2(got1, got[:64]) < 1e-3  # 64 tokens split K over several CTAs: another summation order


# ----------------------------------------------------------------------------- Q8_0, one token (K = 2048 / 4096)
@pytest.mark.parametrize("x_dtype", [DTYPE_F32, DTYPE_BF16])
@pytest.mark.parametrize("out_dtype", [DTYPE_F32, DTYPE_BF16, DTYPE_F16])
@pytest.mark.parametrize("N,K", [(1, 4096), (17, 2048), (4096, 4096), (4747, 4096), (4740, 2048), (30000, 4096),
                                 (20001, 2048)])
def test_q8_0_single_token_kernel(dev, x_dtype, out_dtype, N, K):
    """Eight-row tiles, two CTAs per SM; N not a multiple of 8, fewer and more tiles than CTA slots."""
    rng = np.random.default_rng(N + K)
    w = o.gen_q8_0_weight(rng, N, K)
    x = o.gen_activation(rng, 1, K, x_dtype == DTYPE_BF16)
    want = o.c_qmatmul(x, w, N, K, False)
    got = _run(dev, w, x, 1, N, K, False, x_dtype, out_dtype)
    if out_dtype == DTYPE_F32:
        assert o.rel_l2(got, want) < (1e-4 if N >= 1000 else TOL_DECODE)
    else:
        assert o.rel_l2(got, want) < 4e-3  # storage rounding of y
    assert np.array_equal(got, _run(dev, w, x, 1, N, K, False, x_dtype, out_dtype))  # fixed summation order


def test_q8_0_single_token_extreme_blocks(dev):
    """Weight bytes -128 and 127, activation blocks that are all zero or differ by orders of magnitude."""
    rng = np.random.default_rng(5)
    N, K = 520, 4096
    w = o.gen_q8_0_weight(rng, N, K).reshape(N, K // 32, 34).copy()
    w[:, ::3, 2:] = 0x80   # -128
    w[:, 1::3, 2:] = 0x7F  # 127
    w = w.reshape(-1)
    x = o.gen_activation(rng, 1, K, False)
    x[0, :32] = 0.0
    x[0, 32:64] *= 8192.0
    x[0, 2048:2080] *= 2.0 ** -12
    got = _run(dev, w, x, 1, N, K, False, DTYPE_F32, DTYPE_F32)
    assert o.rel_l2(got, o.c_qmatmul(x, w, N, K, False)) < 1e-4


# ----------------------------------------------------------------------------- two to four tokens (K = 2048 / 4096)
@pytest.mark.parametrize("x_dtype", [DTYPE_F32, DTYPE_BF16])
@pytest.mark.parametrize("out_dtype", [DTYPE_F32, DTYPE_BF16, DTYPE_F16])
@pytest.mark.parametrize("M,N,K", [(2, 1, 4096), (2, 4747, 4096), (3, 17, 2048), (3, 5000, 4096), (4, 4736, 2048),
                                   (4, 30000, 4096), (2, 20000, 2048)])
def test_q4k_two_to_four_tokens(dev, x_dtype, out_dtype, M, N, K):
    """Token pairs in the MMA columns, two CTAs per SM; N not a multiple of 16, more tiles than CTA slots, an odd
    token count (the pair's second token multiplies by zero)."""
    rng = np.random.default_rng(N + K + M)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, x_dtype == DTYPE_BF16)
    want = o.c_qmatmul(x, w, N, K, True)
    got = _run(dev, w, x, M, N, K, True, x_dtype, out_dtype)
    if out_dtype == DTYPE_F32:
        assert o.rel_l2(got, want) < (1e-4 if N >= 1000 else TOL_DECODE)
    else:
        assert o.rel_l2(got, want) < 4e-3  # storage rounding of y
    again = _run(dev, w, x, M, N, K, True, x_dtype, out_dtype)
    assert np.array_equal(got, again)  # fixed summation order


def test_q4k_two_to_four_tokens_rows_differ(dev):
    """Every token meets its own activations: rows of x that differ by orders of magnitude, one all-zero row."""
    rng = np.random.default_rng(99)
    M, N, K = 4, 1000, 4096
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    x[1] *= 4096.0
    x[2] = 0.0
    x[3] *= 2.0 ** -10
    got = _run(dev, w, x, M, N, K, True, DTYPE_BF16, DTYPE_F32)
    want = o.c_qmatmul(x, w, N, K, True)
    for m in (0, 1, 3):
        assert o.rel_l2(got[m], want[m]) < 1e-4, m
    assert not got[2].any()


# ----------------------------------------------------------------------------- five to eight tokens in the MMA columns
@pytest.mark.parametrize("x_dtype,out_dtype", [(DTYPE_BF16, DTYPE_F32), (DTYPE_F32, DTYPE_F32), (DTYPE_BF16, DTYPE_BF16),
                                               (DTYPE_F32, DTYPE_F16)])
@pytest.mark.parametrize("M,N,K", [(5, 1, 4096), (5, 17, 2048), (8, 4747, 4096), (6, 4736, 2048), (7, 30000, 4096),
                                   (8, 20000, 2048), (8, 14336, 4096), (7, 5000, 8192), (8, 130, 8192), (6, 63, 4096)])
def test_q4k_five_to_eight_tokens(dev, x_dtype, out_dtype, M, N, K):
    """Tokens in the columns of the integer MMA, activation fragments shared by the CTAs of a cluster: fewer tiles
    than CTAs (CTAs without a tile still quantise their share), ragged last tile, more tiles per CTA than ring
    stages (30000 rows), 8192-value rows."""
    rng = np.random.default_rng(M + N + K)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, x_dtype == DTYPE_BF16)
    want = o.c_qmatmul(x, w, N, K, True)
    got = _run(dev, w, x, M, N, K, True, x_dtype, out_dtype)
    if out_dtype == DTYPE_F32:
        # 15-bit block fixed-point activations: ~1e-5 over thousands of outputs; a handful of outputs is a handful
        # of samples of that noise, so only the task's tolerance is asserted there
        assert o.rel_l2(got, want) < (1e-4 if M * N >= 1000 else TOL_DECODE)
        assert np.array_equal(got, _run(dev, w, x, M, N, K, True, x_dtype, out_dtype))  # fixed summation order
    else:
        assert np.array_equal(got, o.round_through(_run(dev, w, x, M, N, K, True, x_dtype, DTYPE_F32),
                                                   o.UB_BF16 if out_dtype == DTYPE_BF16 else o.UB_F16))


@pytest.mark.parametrize("M,N,K", [(13, 1000, 4096), (16, 600, 2048), (11, 300, 8192)])
def test_q4k_more_tokens_in_passes_of_eight(dev, M, N, K):
    """Nine to sixteen tokens with f32 on either side: a pass of eight, then five to eight (or the smaller kernels)."""
    rng = np.random.default_rng(M + N + K)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, False)
    got = _run(dev, w, x, M, N, K, True, DTYPE_F32, DTYPE_F32)
    assert o.rel_l2(got, o.c_qmatmul(x, w, N, K, True)) < 1e-4


def test_q4k_five_to_eight_tokens_rows_differ(dev):
    """Every token has its own scale per 256 values: tokens of very different magnitude, a token of zeros, a
    super-block of zeros in one token and a large one in another."""
    rng = np.random.default_rng(77)
    M, N, K = 7, 600, 4096
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    x[1] *= 4096.0
    x[2] *= 1.0 / 1024.0
    x[3] = 0.0
    x[4, :256] = 0.0
    x[5, 256:512] *= 8192.0
    x[6] *= 64.0
    got = _run(dev, w, x, M, N, K, True, DTYPE_BF16, DTYPE_F32)
    want = o.c_qmatmul(x, w, N, K, True)
    for m in range(M):
        if m == 3:
            assert not got[m].any()
        else:
            assert o.rel_l2(got[m], want[m]) < 1e-4, m


# ----------------------------------------------------------------------------- single-token kernel (K = 2048 / 4096)
@pytest.mark.parametrize("x_dtype", [DTYPE_F32, DTYPE_BF16])
@pytest.mark.parametrize("out_dtype", [DTYPE_F32, DTYPE_BF16, DTYPE_F16])
@pytest.mark.parametrize("N,K", [(1, 4096), (17, 2048), (4747, 4096), (4736, 2048), (30000, 4096), (20000, 2048)])
def test_q4k_single_token_kernel(dev, x_dtype, out_dtype, N, K):
    """M = 1 at K = 2048 / 4096: ragged last tile, fewer tiles than CTAs, and more tiles per CTA than the ring has
    stages (30000 rows at K = 4096: 1875 tiles on 296 CTAs of 3 stages, so stages are re-armed)."""
    rng = np.random.default_rng(N + K)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, 1, K, x_dtype == DTYPE_BF16)
    want = o.c_qmatmul(x, w, N, K, True)
    got = _run(dev, w, x, 1, N, K, True, x_dtype, out_dtype)
    if out_dtype == DTYPE_F32:
        # 15-bit block fixed-point activations: ~1e-5 over thousands of rows; a handful of rows is a handful of
        # samples of that noise, so only the task's tolerance is asserted there
        assert o.rel_l2(got, want) < (1e-4 if N >= 1000 else TOL_DECODE)
    else:
        assert np.array_equal(got, o.round_through(_run(dev, w, x, 1, N, K, True, x_dtype, DTYPE_F32),
                                                   o.UB_BF16 if out_dtype == DTYPE_BF16 else o.UB_F16))


def test_q4k_single_token_many_tiles_per_cta(dev):
    """More 16-row tiles per CTA than one batch of partial sums holds (70000 rows: 15 tiles per CTA)."""
    rng = np.random.default_rng(70)
    N, K = 70000, 2048
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, 1, K, True)
    got = _run(dev, w, x, 1, N, K, True, DTYPE_BF16, DTYPE_F32)
    assert o.rel_l2(got, o.c_qmatmul(x, w, N, K, True)) < 1e-4


@pytest.mark.parametrize("K", [2048, 4096])
@pytest.mark.parametrize("N", [4792, 4816, 14336, 5328, 7120])
def test_q4k_single_token_left_over_tiles_in_halves(dev, K, N):
    """Row counts whose 16-row tiles leave a few over after the full rounds of the grid (296 CTAs on 148 SMs): the
    left-over tiles are dealt as 8-row halves.  4792 rows: the last half lies wholly past the matrix; 5328: 37 left over,
    the most that are cut; 7120: more left over than that, so whole tiles again.  A row's arithmetic does not
    depend on which CTA or which half computes it: the last rows equal those of a small matrix of the same bytes."""
    rng = np.random.default_rng(N + K)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, 1, K, True)
    got = _run(dev, w, x, 1, N, K, True, DTYPE_BF16, DTYPE_F32)
    assert o.rel_l2(got, o.c_qmatmul(x, w, N, K, True)) < 1e-4
    tail = 200
    w_tail = np.ascontiguousarray(w.reshape(N, -1)[N - tail:])
    assert np.array_equal(got.reshape(-1)[N - tail:], _run(dev, w_tail, x, 1, tail, K, True, DTYPE_BF16, DTYPE_F32).reshape(-1))


def test_q4k_single_token_zero_and_huge_activations(dev):
    rng = np.random.default_rng(5)
    N, K = 300, 4096
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, 1, K, True)
    x[0, :256] = 0.0                # a whole super-block of zeros (scale 0)
    x[0, 256:512] *= 8192.0         # and one with a large range (a power of two keeps the values bf16)
    got = _run(dev, w, x, 1, N, K, True, DTYPE_BF16, DTYPE_F32)
    assert o.rel_l2(got, o.c_qmatmul(x, w, N, K, True)) < 1e-4


# ----------------------------------------------------------------------------- large K: every kernel the sharded stack uses
@pytest.mark.parametrize("N,K", [(512, 28672), (512, 14336), (640, 8192), (384, 7168), (256, 3584), (8192, 28672),
                                 (5000, 16384), (19200, 14336)])
@pytest.mark.parametrize("M", [1, 2])
def test_q4k_decode_large_k(dev, M, N, K):
    """Row lengths of the 70B-shaped stack and of its tensor-parallel shards (down projection 28672 / tp; others
    8192).  One token beyond 12288 values runs in passes over K (four at 28672, two at 14336 / 16384) as long as a
    CTA's tiles fit one batch (19200 rows do not: the streaming kernel); two tokens take the older kernels."""
    rng = np.random.default_rng(K + M)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    got = _run(dev, w, x, M, N, K, True, DTYPE_BF16, DTYPE_F32)
    want = o.c_qmatmul(x, w, N, K, True)
    assert o.rel_l2(got, want) < TOL_DECODE
    if M == 1:
        assert o.rel_l2(got, want) < 1e-4
        assert np.array_equal(got, _run(dev, w, x, M, N, K, True, DTYPE_BF16, DTYPE_F32))
        got32 = _run(dev, w, x.astype(np.float32), M, N, K, True, DTYPE_F32, DTYPE_F32)  # f32 activations
        assert o.rel_l2(got32, want) < 1e-4


@pytest.mark.parametrize("is_q4k,M,N,K", [(True, 4, 48, 12544), (False, 4, 40, 16640), (True, 3, 33, 12800),
                                          (False, 2, 19, 16896)])
def test_decode_rows_too_long_for_the_staged_kernels(dev, is_q4k, M, N, K):
    """Several tokens with rows whose activations fit none of the staged kernels' shared-memory plans: the plain
    warp-per-row kernels (the last fallback of the dispatch) compute them."""
    rng = np.random.default_rng(K + M)
    w = (o.gen_q4k_weight if is_q4k else o.gen_q8_0_weight)(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    got = _run(dev, w, x, M, N, K, is_q4k, DTYPE_BF16, DTYPE_F32)
    assert o.rel_l2(got, o.c_qmatmul(x, w, N, K, is_q4k)) < 1e-4


# ----------------------------------------------------------------------------- weights written just before the matmul
def test_quantize_then_matmul_back_to_back(dev):
    """ub_quantize_q8_0 and the Q8_0 matmul on one stream with nothing in between: the matmul must not request
    weight tiles ahead of its dependency wait."""
    rng = np.random.default_rng(8)
    N, K = 4096, 4096
    wf = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    x = o.gen_activation(rng, 1, K, False)
    want = o.c_qmatmul(x, o.c_quantize_q8_0(wf.reshape(-1)), N, K, False)
    d_wf, d_x = dev.htod_sync_copy(wf), dev.htod_sync_copy(x)
    d_y = dev.alloc(N * 4)
    for rep in range(3):  # a fresh destination every time, so that stale bytes cannot pass
        d_wq = dev.alloc_zeros(N * K // 32 * 34)
        dev.synchronize()
        ops.quantize_q8_0(d_wq, d_wf, N * K, DTYPE_F32, stream=dev.stream)
        ops.qmatmul(d_y, d_x, d_wq, 1, N, K, is_q4k=False, x_dtype=DTYPE_F32, out_dtype=DTYPE_F32, stream=dev.stream)
        got = dev.dtoh_sync_copy(d_y, np.float32, (1, N))
        assert o.rel_l2(got, want) < 1e-4


@pytest.mark.parametrize("M,K", [(1, 4096), (2, 4096), (1, 8192), (6, 4096)])
def test_repack_then_q4k_matmul_back_to_back(dev, M, K):
    from ubridge_b200._lib import UB_QMATMUL_WEIGHTS_FRESH

    rng = np.random.default_rng(9)
    N = 2048
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    want = o.c_qmatmul(x, w, N, K, True)
    nblocks = N * K // 256
    d_w = dev.htod_sync_copy(w)
    d_split = dev.alloc(w.size)
    ops.repack_to_split(d_split, d_w, nblocks, True, stream=dev.stream)
    d_x = dev.htod_sync_copy(to_storage(x, DTYPE_BF16))
    d_y = dev.alloc(M * N * 4)
    for flag in (0, UB_QMATMUL_WEIGHTS_FRESH):
        d_w2 = dev.alloc_zeros(w.size)
        dev.synchronize()
        ops.repack_to_interleaved(d_w2, d_split, nblocks, True, stream=dev.stream)
        ops.qmatmul(d_y, d_x, d_w2, M, N, K, is_q4k=True, x_dtype=DTYPE_BF16, out_dtype=DTYPE_F32 | flag,
                    stream=dev.stream)
        got = dev.dtoh_sync_copy(d_y, np.float32, (M, N))
        assert o.rel_l2(got, want) < 1e-4


@pytest.mark.parametrize("M", [16, 40])
def test_repack_then_tensor_core_matmul_back_to_back(dev, M):
    """The K-split launches request their first weight tiles ahead of the dependency wait unless the weights are
    fresh: the library tracks its own weight-writing entry points, callers with their own pass the flag."""
    from ubridge_b200._lib import UB_QMATMUL_WEIGHTS_FRESH

    rng = np.random.default_rng(19)
    N, K = 2048, 4096
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, M, K, True)
    want = x @ o.c_dequant(w, True).reshape(N, K).T
    nblocks = N * K // 256
    d_w = dev.htod_sync_copy(w)
    d_split = dev.alloc(w.size)
    ops.repack_to_split(d_split, d_w, nblocks, True, stream=dev.stream)
    d_x = dev.htod_sync_copy(to_storage(x, DTYPE_BF16))
    d_y = dev.alloc(M * N * 2)
    for flag in (0, UB_QMATMUL_WEIGHTS_FRESH):
        d_w2 = dev.alloc_zeros(w.size)
        dev.synchronize()
        ops.repack_to_interleaved(d_w2, d_split, nblocks, True, stream=dev.stream)
        ops.qmatmul(d_y, d_x, d_w2, M, N, K, is_q4k=True, x_dtype=DTYPE_BF16, out_dtype=DTYPE_BF16 | flag,
                    stream=dev.stream)
        assert o.rel_l2(fetch(dev, d_y, DTYPE_BF16, (M, N)), want) < 5e-3


@pytest.mark.parametrize("x_dtype", [DTYPE_F32, DTYPE_BF16])
@pytest.mark.parametrize("N,K", [(33, 8192), (5000, 8192), (20000, 6144), (4100, 12288), (9000, 10240)])
def test_q4k_single_token_long_rows(dev, x_dtype, N, K):
    """M = 1 with K a multiple of 2048 beyond 4096: the activation fragments live in shared memory, a tile takes
    K / 2048 stages, stages are re-armed many times (20000 rows at K = 6144: 13 stages per CTA through a ring of 4)."""
    rng = np.random.default_rng(N + K)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, 1, K, x_dtype == DTYPE_BF16)
    got = _run(dev, w, x, 1, N, K, True, x_dtype, DTYPE_F32)
    assert o.rel_l2(got, o.c_qmatmul(x, w, N, K, True)) < (1e-4 if N >= 1000 else TOL_DECODE)


# ----------------------------------------------------------------------------- gate/up with SiLU.up in the epilogue
@pytest.mark.parametrize("M,I,K", [(1, 1000, 2048), (1, 4744, 8192), (1, 37, 4096), (1, 640, 1024), (3, 520, 2048),
                                   (40, 264, 1024)])
def test_gate_up_silu_matches_the_two_call_sequence(dev, M, I, K):
    """One token with K % 2048 == 0 is one launch; the result must have the bits of matmul -> ub_silu_and_mul
    (which every other shape runs)."""
    rng = np.random.default_rng(M + I + K)
    w = o.gen_q4k_weight(rng, 2 * I, K)
    x = o.gen_activation(rng, M, K, True)
    d_w, d_x = dev.htod_sync_copy(w), dev.htod_sync_copy(to_storage(x, DTYPE_BF16))
    ws_bytes = ops.qmatmul_q4k_gate_up_workspace_bytes(M, I, K)
    ws = dev.alloc(max(ws_bytes, 256))
    d_y = dev.alloc(M * I * 2)
    ops.qmatmul_q4k_gate_up(d_y, d_x, d_w, M, I, K, out_dtype=DTYPE_BF16, workspace=ws, ws_bytes=ws_bytes,
                            stream=dev.stream)
    got = fetch(dev, d_y, DTYPE_BF16, (M, I))
    # the two-call sequence on the device
    d_gu, d_y2 = dev.alloc(M * 2 * I * 2), dev.alloc(M * I * 2)
    ws2_bytes = ops.qmatmul_workspace_bytes(M, 2 * I, K, True)
    ws2 = dev.alloc(max(ws2_bytes, 256))
    ops.qmatmul(d_gu, d_x, d_w, M, 2 * I, K, is_q4k=True, x_dtype=DTYPE_BF16, out_dtype=DTYPE_BF16, workspace=ws2,
                ws_bytes=ws2_bytes, stream=dev.stream)
    ops.silu_and_mul(d_y2, d_gu, M, I, DTYPE_BF16, stream=dev.stream)
    assert np.array_equal(got, fetch(dev, d_y2, DTYPE_BF16, (M, I)))
    # and the oracle: exact matmul, rounded to bf16, SiLU.up
    gu = o.round_through(o.c_qmatmul(x, w, 2 * I, K, True), o.UB_BF16)
    want = o.silu_and_mul(gu, o.UB_BF16)
    assert o.rel_l2(got, want) < (1e-2 if M > 8 else 5e-3)


# ----------------------------------------------------------------------------- RMSNorm in front, residual behind
@pytest.mark.parametrize("dtype", [DTYPE_F32, DTYPE_F16, DTYPE_BF16])
def test_rms_norm_standalone(dev, dtype):
    rng = np.random.default_rng(21)
    T, H = 7, 1000
    x = o.round_through(rng.standard_normal((T, H)).astype(np.float32) * 3, {DTYPE_F32: o.UB_F32, DTYPE_F16: o.UB_F16, DTYPE_BF16: o.UB_BF16}[dtype])
    g = o.round_through(rng.uniform(0.5, 1.5, size=H).astype(np.float32), {DTYPE_F32: o.UB_F32, DTYPE_F16: o.UB_F16, DTYPE_BF16: o.UB_BF16}[dtype])
    want = o.rms_norm(x, g, 1e-5, {DTYPE_F32: o.UB_F32, DTYPE_F16: o.UB_F16, DTYPE_BF16: o.UB_BF16}[dtype])
    d_out = dev.alloc(T * H * ESIZE[dtype])
    ops.rms_norm(d_out, dev.htod_sync_copy(to_storage(x, dtype)), dev.htod_sync_copy(to_storage(g, dtype)), T, H, 1e-5,
                 dtype, stream=dev.stream)
    got = fetch(dev, d_out, dtype, (T, H))
    # f32 vs f64 mean and rsqrt: a value on a rounding boundary may fall the other way, by one unit of the type
    assert o.rel_l2(got, want) < {DTYPE_F32: 1e-6, DTYPE_F16: 1e-3, DTYPE_BF16: 4e-3}[dtype]


@pytest.mark.parametrize("M,N,K,gate_up", [(1, 1000, 4096, False), (1, 640, 2048, False), (1, 520, 8192, False),
                                           (1, 4816, 4096, False), (1, 2408, 4096, True),
                                           (1, 700, 8192, True), (1, 96, 1024, False), (3, 200, 2048, True),
                                           (20, 136, 1024, False)])
def test_matmul_on_rms_norm(dev, M, N, K, gate_up):
    """ub_qmatmul_q4k_rmsnorm_bf16: one launch for one token (the norm in the matmul's prologue), norm + matmul
    otherwise; against the oracle's norm -> exact matmul (-> SiLU.up)."""
    rng = np.random.default_rng(M + N + K)
    rows = 2 * N if gate_up else N
    w = o.gen_q4k_weight(rng, rows, K)
    x = o.gen_activation(rng, M, K, True) * 2.5
    x = o.round_through(x, o.UB_BF16)
    g = o.round_through(rng.uniform(0.5, 1.5, size=K).astype(np.float32), o.UB_BF16)
    xn = o.rms_norm(x, g, 1e-5, o.UB_BF16)
    full = o.c_qmatmul(xn, w, rows, K, True)
    want = o.silu_and_mul(o.round_through(full, o.UB_BF16), o.UB_BF16) if gate_up else full
    ws_bytes = ops.qmatmul_q4k_rmsnorm_workspace_bytes(M, N, K, gate_up)
    ws = dev.alloc(max(ws_bytes, 256))
    d_y = dev.alloc(M * N * 2)
    ops.qmatmul_q4k_rmsnorm(d_y, dev.htod_sync_copy(to_storage(x, DTYPE_BF16)), dev.htod_sync_copy(to_storage(g, DTYPE_BF16)),
                            1e-5, dev.htod_sync_copy(w), M, N, K, gate_up=gate_up, out_dtype=DTYPE_BF16, workspace=ws,
                            ws_bytes=ws_bytes, stream=dev.stream)
    got = fetch(dev, d_y, DTYPE_BF16, (M, N))
    # bf16 activations after the norm (a boundary case may round the other way) and bf16 output
    assert o.rel_l2(got, want) < 8e-3


@pytest.mark.parametrize("N,K", [(1024, 4096), (520, 8192), (200, 1024), (4816, 4096)])
def test_matmul_with_residual_on_one_rank(dev, N, K):
    import ctypes

    from ubridge_b200._lib import check, lib

    rng = np.random.default_rng(N + K)
    w = o.gen_q4k_weight(rng, N, K)
    x = o.gen_activation(rng, 1, K, True)
    r = o.round_through(rng.standard_normal((1, N)).astype(np.float32), o.UB_BF16)
    want = r + o.c_qmatmul(x, w, N, K, True)
    d_y = dev.alloc(N * 2)
    d = [dev.htod_sync_copy(v) for v in (to_storage(x, DTYPE_BF16), w, to_storage(r, DTYPE_BF16))]
    check(lib().ub_qmatmul_q4k_allreduce_residual_bf16(ctypes.c_void_p(d_y.ptr), ctypes.c_void_p(d[0].ptr),
                                                       ctypes.c_void_p(d[1].ptr), ctypes.c_void_p(d[2].ptr), 1, N, K,
                                                       None, 0, 1, 0, dev.stream), "residual matmul")
    got = fetch(dev, d_y, DTYPE_BF16, (1, N))
    assert o.rel_l2(got, want) < 5e-3
