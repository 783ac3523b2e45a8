"""GPU parity: router, alignment, grouped expert GEMMs, combine and the whole Q4_K expert layer."""
import numpy as np
import pytest

from oracle import oracle as o
from ubridge_b200 import DTYPE_BF16, DTYPE_F16, DTYPE_F32, ops
from ubridge_b200._lib import UB_ERR_BAD_INDEX

from _util import ESIZE, NP_STORAGE, fetch, from_storage, to_storage

pytestmark = pytest.mark.gpu

ODT = {DTYPE_F32: o.UB_F32, DTYPE_F16: o.UB_F16, DTYPE_BF16: o.UB_BF16}


# ----------------------------------------------------------------------------- router
@pytest.mark.parametrize("dtype", [DTYPE_F32, DTYPE_F16, DTYPE_BF16])
@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (256, 8, 2), (37, 64, 6), (5, 128, 8), (3, 300, 4), (2, 4096, 3)])
@pytest.mark.parametrize("norm", [False, True])
def test_topk_softmax(dev, dtype, T, E, k, norm):
    rng = np.random.default_rng(T * 31 + E)
    lg = to_storage(rng.standard_normal((T, E)).astype(np.float32), dtype)
    lg_f32 = from_storage(lg, dtype)
    want_w, want_i = o.topk_softmax(lg_f32, k, norm, ODT[dtype])
    d_l = dev.htod_sync_copy(lg)
    d_w = dev.alloc(T * k * ESIZE[dtype])
    d_i = dev.alloc(T * k * 4)
    ops.topk_softmax(d_l, d_w, d_i, T, E, k, norm, dtype, stream=dev.stream)
    got_i = dev.dtoh_sync_copy(d_i, np.int32, (T, k))
    got_w = fetch(dev, d_w, dtype, (T, k))
    # indices exact unless two probabilities are equal to the last bit (then the same weight either way)
    same = got_i == want_i
    if not same.all():
        p = np.exp(lg_f32 - lg_f32.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        rows, cols = np.nonzero(~same)
        assert np.allclose(p[rows, got_i[rows, cols]], p[rows, want_i[rows, cols]], rtol=1e-6)
    # <= 1 ulp of T for the 16-bit types; for f32 the device expf and libm's differ by a couple of ulps
    ulp = {DTYPE_F32: 1e-6, DTYPE_F16: 2.0 ** -10, DTYPE_BF16: 2.0 ** -7}[dtype]
    assert np.allclose(got_w, want_w, rtol=ulp, atol=1e-30)


def test_topk_softmax_ties_and_c_oracle_agree(dev):
    lg = np.array([[1, 3, 3, 0, 3, -1, 0, 0], [2] * 8], dtype=np.float32)
    d_l = dev.htod_sync_copy(lg)
    d_w, d_i = dev.alloc(2 * 3 * 4), dev.alloc(2 * 3 * 4)
    ops.topk_softmax(d_l, d_w, d_i, 2, 8, 3, False, DTYPE_F32, stream=dev.stream)
    assert dev.dtoh_sync_copy(d_i, np.int32, (2, 3)).tolist() == [[1, 2, 4], [0, 1, 2]]
    cw, ci = o.c_topk_softmax(lg, 3, False, o.UB_F32)
    assert ci.tolist() == [[1, 2, 4], [0, 1, 2]]
    assert np.allclose(dev.dtoh_sync_copy(d_w, np.float32, (2, 3)), cw, rtol=1e-6)


# ----------------------------------------------------------------------------- alignment
def _align(dev, ids, E, block, real=None, emap=None):
    T, k = ids.shape
    n_sorted, n_blocks = ops.moe_align_sizes(T, k, E, block)
    d_ids = dev.htod_sync_copy(ids.astype(np.int32))
    d_s, d_e, d_n = dev.alloc(max(n_sorted, 1) * 4), dev.alloc(max(n_blocks, 1) * 4), dev.alloc(4)
    d_r = dev.htod_sync_copy(np.array([real], dtype=np.int32)) if real is not None else None
    d_m = dev.htod_sync_copy(np.asarray(emap, dtype=np.int32)) if emap is not None else None
    ops.moe_align_block_size(d_s, d_e, d_n, d_ids, E, block, T, k, real_token_num=d_r, expert_map=d_m,
                             stream=dev.stream)
    s = dev.dtoh_sync_copy(d_s, np.int32)[:n_sorted]
    e = dev.dtoh_sync_copy(d_e, np.int32)[:n_blocks]
    n = int(dev.dtoh_sync_copy(d_n, np.int32)[0])
    return s, e, n


@pytest.mark.parametrize("T,k,E,block", [(256, 2, 8, 64), (1, 2, 8, 64), (3, 1, 4, 2), (513, 4, 60, 16),
                                         (2048, 8, 256, 64), (4096, 2, 8, 128), (33, 2, 1000, 8)])
def test_moe_align_matches_oracle(dev, T, k, E, block):
    rng = np.random.default_rng(T + E)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    want = o.c_moe_align(ids, E, block)
    got = _align(dev, ids, E, block)
    assert got[2] == want[2]
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_moe_align_edge_cases(dev):
    ids = np.array([[0, 2], [2, 0], [2, 2]])
    s, e, n = _align(dev, ids, 3, 2)
    assert s.tolist() == [0, 3, 1, 2, 4, 5, 6, 6, 6] and e.tolist() == [0, 2, 2, 0] and n == 6
    s, e, n = _align(dev, np.array([[1, 1], [1, 1]]), 2, 3)                       # all tokens to one expert
    assert s.tolist() == [0, 1, 2, 3, 4, 4, 4, 4] and e.tolist() == [1, 1] and n == 6
    ids = np.array([[0, 1], [1, 2], [2, 0], [3, 3]])
    s, e, n = _align(dev, ids, 4, 2, emap=[-1, 0, 1, -1])                        # expert-parallel map
    assert s[:8].tolist() == [0, 5, 1, 2, 3, 4, 6, 7] and e[:4].tolist() == [-1, 0, 1, -1] and n == 8
    s, e, n = _align(dev, ids, 4, 2, real=2)                                     # device-side token count
    assert s[:6].tolist() == [0, 8, 1, 2, 3, 8] and e[:3].tolist() == [0, 1, 2] and n == 6
    s, e, n = _align(dev, ids, 4, 2, real=0)
    assert n == 0 and (s == 8).all() and (e == 0).all()


def test_moe_align_bad_id_sets_error_word_instead_of_trapping(dev):
    ids = np.array([[0, 9], [1, 2]])
    assert dev.device_status() == 0
    s, e, n = _align(dev, ids, 4, 2)
    assert dev.device_status() == UB_ERR_BAD_INDEX   # read-and-clear
    assert dev.device_status() == 0
    # the valid slots are still placed
    assert s[:6].tolist() == [0, 4, 2, 4, 3, 4] and n == 6


# ----------------------------------------------------------------------------- dense grouped GEMM (reference signature)
@pytest.mark.parametrize("dtype", [DTYPE_F16, DTYPE_BF16])
@pytest.mark.parametrize("T,H,N,E,k,block", [(9, 64, 40, 4, 2, 4), (64, 128, 96, 8, 2, 16), (130, 256, 72, 6, 3, 64),
                                             (40, 72, 33, 3, 1, 128)])
@pytest.mark.parametrize("mul", [0, 1])
def test_invoke_fused_moe_dense(dev, dtype, T, H, N, E, k, block, mul):
    rng = np.random.default_rng(T + N + mul)
    rows_a = T * k if mul else T
    A = from_storage(to_storage(rng.standard_normal((rows_a, H)).astype(np.float32), dtype), dtype)
    B = from_storage(to_storage((rng.standard_normal((E, N, H)) * 0.2).astype(np.float32), dtype), dtype)
    bias = from_storage(to_storage(rng.standard_normal((E, N)).astype(np.float32), dtype), dtype)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    w = rng.uniform(0.1, 1, size=(T, k)).astype(np.float32)
    s, e, npp = o.c_moe_align(ids, E, block)
    for bias_flag in (0, 1):
        want = o.fused_moe(A, B, w, s, e, npp, k, block, mul, ODT[dtype], T * k, bias=bias if bias_flag else None)
        d = {n_: dev.htod_sync_copy(v) for n_, v in dict(A=to_storage(A, dtype), B=to_storage(B, dtype),
                                                           bias=to_storage(bias, dtype), w=w, s=s, e=e,
                                                           n=np.array([npp], dtype=np.int32)).items()}
        d_C = dev.alloc_zeros(T * k * N * 2)
        ops.invoke_fused_moe(d_C, d["A"], d["B"], d["bias"], d["w"], d["s"], d["e"], d["n"], T, H, N, E, T * k, k,
                             block, bool(mul), bool(bias_flag), dtype, stream=dev.stream)
        got = fetch(dev, d_C, dtype, (T * k, N))
        assert o.rel_l2(got, want) < 2e-3  # f32 vs f64 accumulation, then one rounding to T


def test_invoke_fused_moe_expert_minus_one_and_empty(dev):
    rng = np.random.default_rng(3)
    T, H, N, E, k, block = 12, 64, 24, 4, 2, 4
    A = o.gen_activation(rng, T, H, True)
    B = o.bf16_bits_to_f32(o.f32_to_bf16_bits((rng.standard_normal((2, N, H)) * 0.2).astype(np.float32)))
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    emap = np.array([0, -1, 1, -1], dtype=np.int32)
    s, e, npp = o.c_moe_align(ids, E, block, expert_map=emap)
    C0 = np.full((T * k, N), 7.0, dtype=np.float32)
    want = o.fused_moe(A, B, None, s, e, npp, k, block, 0, o.UB_BF16, T * k, C_init=C0)
    d_C = dev.htod_sync_copy(to_storage(C0, DTYPE_BF16))
    args = [dev.htod_sync_copy(v) for v in (to_storage(A, DTYPE_BF16), to_storage(B, DTYPE_BF16), s, e)]
    d_n = dev.htod_sync_copy(np.array([npp], dtype=np.int32))
    ops.invoke_fused_moe(d_C, args[0], args[1], None, None, args[2], args[3], d_n, T, H, N, E, T * k, k, block, False,
                         False, DTYPE_BF16, stream=dev.stream)
    got = fetch(dev, d_C, DTYPE_BF16, (T * k, N))
    assert o.rel_l2(got, want) < 2e-3
    flat = ids.reshape(-1)
    assert all((got[i] == 0).all() for i in range(T * k) if emap[flat[i]] == -1)
    # num_tokens_post_pad == 0: nothing is written (kernels/fused_moe_host.cpp:89-93)
    d_C2 = dev.htod_sync_copy(to_storage(C0, DTYPE_BF16))
    d_zero = dev.htod_sync_copy(np.array([0], dtype=np.int32))
    ops.invoke_fused_moe(d_C2, args[0], args[1], None, None, args[2], args[3], d_zero, T, H, N, E, T * k, k, block,
                         False, False, DTYPE_BF16, stream=dev.stream)
    assert (fetch(dev, d_C2, DTYPE_BF16, (T * k, N)) == 7.0).all()


# ----------------------------------------------------------------------------- combine, indexed, elementwise
@pytest.mark.parametrize("dtype", [DTYPE_F16, DTYPE_BF16])
def test_moe_combine(dev, dtype):
    rng = np.random.default_rng(6)
    N, K, M, topk = 37, 90, 520, 4
    y0 = from_storage(to_storage(rng.standard_normal((N, M)).astype(np.float32), dtype), dtype)
    e_out = to_storage(rng.standard_normal((K, M)).astype(np.float32), dtype)
    w = rng.uniform(0, 1, size=(N, topk)).astype(np.float32)
    idx = rng.integers(0, N + 3, size=K).astype(np.uint32)   # a few rows out of range: skipped
    top = rng.integers(0, topk + 1, size=K).astype(np.uint32)  # a few slots out of range: skipped
    y_host = to_storage(y0, dtype).copy()
    o.clib().ub_oracle_moe_combine(o._p(y_host), o._p(e_out), o._p(w), o._p(idx), o._p(top), N, K, M, topk, ODT[dtype])
    d_y = dev.htod_sync_copy(to_storage(y0, dtype))
    d = [dev.htod_sync_copy(v) for v in (e_out, w, idx, top)]
    ops.moe_combine(d_y, d[0], d[1], d[2], d[3], N, K, M, topk, dtype, stream=dev.stream)
    got = dev.dtoh_sync_copy(d_y, NP_STORAGE[dtype], (N, M))
    assert np.array_equal(got.view(np.uint16), y_host.view(np.uint16))  # same roundings in the same order


@pytest.mark.parametrize("dtype", [DTYPE_F16, DTYPE_BF16])
@pytest.mark.parametrize("M_is_topk", [False, True])
def test_indexed_moe(dev, dtype, M_is_topk):
    rng = np.random.default_rng(8)
    batch, topk, N, K, E = 5, 3, 40, 256, 6
    M = topk if M_is_topk else 1
    x = to_storage(rng.standard_normal((batch, M, K)).astype(np.float32), dtype)
    w = to_storage((rng.standard_normal((E, N, K)) * 0.1).astype(np.float32), dtype)
    idx = rng.integers(0, E, size=(batch, topk)).astype(np.uint32)
    want = np.zeros((batch, topk, N), dtype=NP_STORAGE[dtype])
    wf = np.ascontiguousarray(from_storage(w, dtype))
    o.clib().ub_oracle_indexed_moe(o._p(x), o._p(wf), o._p(want), o._p(idx), N, K, M, batch, topk, E, ODT[dtype])
    d = [dev.htod_sync_copy(v) for v in (x, w, idx)]
    d_out = dev.alloc(batch * topk * N * 2)
    ops.indexed_moe(d[0], d[1], d_out, d[2], N, K, M, batch, topk, E, dtype, stream=dev.stream)
    got = fetch(dev, d_out, dtype, (batch, topk, N))
    assert o.rel_l2(got, from_storage(want, dtype)) < 2e-3


@pytest.mark.parametrize("dtype", [DTYPE_F16, DTYPE_BF16])
@pytest.mark.parametrize("batch,topk,N,K,E,M_is_topk", [(5, 3, 200, 1024, 6, False), (12, 2, 333, 4096, 8, False),
                                                       (3, 4, 64, 512, 5, True), (1, 2, 1, 256, 2, True)])
def test_indexed_moe_q4k(dev, dtype, batch, topk, N, K, E, M_is_topk):
    """indexed_moe on Q4_K experts: per (token, slot) the exact matrix-vector product against that slot's expert
    (the oracle's dequantised weights, f32 accumulation), rounded once to the storage type."""
    rng = np.random.default_rng(batch + N + K)
    M = topk if M_is_topk else 1
    x = from_storage(to_storage(rng.standard_normal((batch, M, K)).astype(np.float32), dtype), dtype)
    w = o.gen_q4k_weight(rng, E * N, K)
    wb = w.reshape(E, -1)
    idx = rng.integers(0, E, size=(batch, topk)).astype(np.uint32)
    want = np.zeros((batch, topk, N), dtype=np.float32)
    for b in range(batch):
        for t in range(topk):
            xr = x[b, 0 if M == 1 else t][None, :]
            want[b, t] = o.c_qmatmul(xr, wb[idx[b, t]], N, K, True)[0]
    d = [dev.htod_sync_copy(v) for v in (to_storage(x, dtype), w, idx)]
    d_out = dev.alloc(batch * topk * N * 2)
    ops.indexed_moe_q4k(d_out, d[0], d[1], d[2], N, K, M, batch, topk, E, dtype, stream=dev.stream)
    got = fetch(dev, d_out, dtype, (batch, topk, N))
    assert o.rel_l2(got, want) < 3e-3  # exact f32 products, one rounding to the 16-bit output
    assert np.array_equal(got, o.round_through(want, ODT[dtype])) or o.rel_l2(got, o.round_through(want, ODT[dtype])) < 1e-3


def test_indexed_moe_q4k_bad_index_gives_zero_row_and_error_word(dev):
    rng = np.random.default_rng(4)
    batch, topk, N, K, E = 2, 2, 70, 256, 3
    x = to_storage(rng.standard_normal((batch, 1, K)).astype(np.float32), DTYPE_BF16)
    w = o.gen_q4k_weight(rng, E * N, K)
    idx = np.array([[0, 7], [2, 1]], dtype=np.uint32)
    d = [dev.htod_sync_copy(v) for v in (x, w, idx)]
    d_out = dev.htod_sync_copy(np.full(batch * topk * N, 0x7FC0, dtype=np.uint16))
    assert dev.device_status() == 0
    ops.indexed_moe_q4k(d_out, d[0], d[1], d[2], N, K, 1, batch, topk, E, DTYPE_BF16, stream=dev.stream)
    got = fetch(dev, d_out, DTYPE_BF16, (batch, topk, N))
    assert dev.device_status() == UB_ERR_BAD_INDEX
    assert (got[0, 1] == 0).all() and np.isfinite(got).all() and np.abs(got[1]).max() > 0


def test_silu_and_mul_and_topk_sum(dev):
    rng = np.random.default_rng(12)
    x = o.gen_activation(rng, 33, 2 * 72, True) * 4
    d_x = dev.htod_sync_copy(to_storage(x, DTYPE_BF16))
    d_o = dev.alloc(33 * 72 * 2)
    ops.silu_and_mul(d_o, d_x, 33, 72, DTYPE_BF16, stream=dev.stream)
    got = fetch(dev, d_o, DTYPE_BF16, (33, 72))
    want = o.silu_and_mul(x, o.UB_BF16)
    assert np.allclose(got, want, rtol=2 ** -7, atol=1e-30)  # expf differs by an ulp between libm and CUDA
    assert (got == want).mean() > 0.98
    y = o.gen_activation(rng, 20 * 3, 64, True)
    d_y = dev.htod_sync_copy(to_storage(y, DTYPE_BF16))
    d_s = dev.alloc(20 * 64 * 2)
    ops.topk_sum(d_s, d_y, 20, 3, 64, DTYPE_BF16, stream=dev.stream)
    assert np.array_equal(fetch(dev, d_s, DTYPE_BF16, (20, 64)), o.topk_sum(y, 20, 3, o.UB_BF16))


# ----------------------------------------------------------------------------- Q4_K grouped GEMM and the whole layer
def _moe_problem(seed, T, H, I, E, k):
    rng = np.random.default_rng(seed)
    w13 = o.gen_q4k_weight(rng, E * 2 * I, H)
    w2 = o.gen_q4k_weight(rng, E * H, I)
    hidden = o.gen_activation(rng, T, H, True)
    logits = o.gen_activation(rng, T, E, True)
    return w13, w2, hidden, logits


@pytest.mark.parametrize("T,H,I,E,k,block", [(7, 256, 256, 4, 2, 4), (40, 512, 768, 8, 2, 16), (130, 256, 512, 6, 3, 64)])
def test_fused_moe_q4k_gemm_both_flavours(dev, T, H, I, E, k, block):
    w13, w2, hidden, logits = _moe_problem(T, T, H, I, E, k)
    tw, ti = o.topk_softmax(logits, k, True, o.UB_BF16)
    s, e, npp = o.c_moe_align(ti, E, block)
    w13d = o.c_dequant(w13, True).reshape(E, 2 * I, H)
    w2d = o.c_dequant(w2, True).reshape(E, H, I)
    c1 = o.fused_moe(hidden, w13d, None, s, e, npp, k, block, 0, o.UB_BF16, T * k)
    act = o.silu_and_mul(c1, o.UB_BF16)
    c2 = o.fused_moe(act, w2d, tw, s, e, npp, k, block, 1, o.UB_BF16, T * k)
    d = {n_: dev.htod_sync_copy(v) for n_, v in dict(w13=w13, w2=w2, h=to_storage(hidden, DTYPE_BF16), tw=tw, s=s, e=e,
                                                       n=np.array([npp], dtype=np.int32)).items()}
    # plain flavour: C1 [T*k, 2I]
    d_c1 = dev.alloc_zeros(T * k * 2 * I * 2)
    ops.fused_moe_q4k_gemm(d_c1, d["h"], d["w13"], None, d["s"], d["e"], d["n"], T, H, 2 * I, E, T * k, k, block, False,
                           False, stream=dev.stream)
    assert o.rel_l2(fetch(dev, d_c1, DTYPE_BF16, (T * k, 2 * I)), c1) < 1e-2
    # fused SiLU.up flavour: act [T*k, I]
    d_act = dev.alloc_zeros(T * k * I * 2)
    ops.fused_moe_q4k_gemm(d_act, d["h"], d["w13"], None, d["s"], d["e"], d["n"], T, H, 2 * I, E, T * k, k, block,
                           False, True, stream=dev.stream)
    got_act = fetch(dev, d_act, DTYPE_BF16, (T * k, I))
    assert o.rel_l2(got_act, act) < 1e-2
    # second GEMM with the routed weight, fed with the oracle's activations
    d_a = dev.htod_sync_copy(to_storage(act, DTYPE_BF16))
    d_c2 = dev.alloc_zeros(T * k * H * 2)
    ops.fused_moe_q4k_gemm(d_c2, d_a, d["w2"], d["tw"], d["s"], d["e"], d["n"], T * k, I, H, E, T * k, k, block, True,
                           False, stream=dev.stream)
    assert o.rel_l2(fetch(dev, d_c2, DTYPE_BF16, (T * k, H)), c2) < 1e-2


@pytest.mark.parametrize("T,H,I,E,k,block", [(7, 256, 256, 4, 2, 4), (64, 512, 768, 8, 2, 64)])
def test_moe_layer_q4k_small(dev, T, H, I, E, k, block):
    w13, w2, hidden, logits = _moe_problem(50 + T, T, H, I, E, k)
    want, _ = o.moe_layer_exact(hidden, logits, o.c_dequant(w13, True).reshape(E, 2 * I, H),
                                o.c_dequant(w2, True).reshape(E, H, I), k, block, True)
    d = [dev.htod_sync_copy(v) for v in (to_storage(hidden, DTYPE_BF16), to_storage(logits, DTYPE_BF16), w13, w2)]
    ws_bytes = ops.moe_layer_q4k_workspace_bytes(T, H, I, E, k, block)
    ws, d_out = dev.alloc(ws_bytes), dev.alloc(T * H * 2)
    ops.moe_layer_q4k(d_out, d[0], d[1], d[2], d[3], T, H, I, E, k, block, True, ws, ws_bytes, stream=dev.stream)
    assert o.rel_l2(fetch(dev, d_out, DTYPE_BF16, (T, H)), want) < 1e-2


def test_moe_layer_q4k_expert_parallel_partials_sum_to_the_whole(dev):
    from ubridge_b200 import parallel as par
    T, H, I, E, k, block = 24, 256, 512, 4, 2, 8
    w13, w2, hidden, logits = _moe_problem(99, T, H, I, E, k)
    want, _ = o.moe_layer_exact(hidden, logits, o.c_dequant(w13, True).reshape(E, 2 * I, H),
                                o.c_dequant(w2, True).reshape(E, H, I), k, block, True)
    d_h, d_l = dev.htod_sync_copy(to_storage(hidden, DTYPE_BF16)), dev.htod_sync_copy(to_storage(logits, DTYPE_BF16))
    total = np.zeros((T, H), dtype=np.float32)
    w13b = w13.reshape(E, -1)
    w2b = w2.reshape(E, -1)
    for rank in range(2):
        e0, e1 = par.expert_range(E, rank, 2)
        layer = par.EPMoELayer(dev, T, H, I, E, k, block, rank, 2, w13b[e0:e1], w2b[e0:e1])
        total += fetch(dev, layer.forward(d_h, d_l), DTYPE_BF16, (T, H))
    assert o.rel_l2(total, want) < 1e-2


def test_config4_mixtral_layer_full_size(dev):
    """8 experts, top-2, hidden 4096, intermediate 14336, 256 tokens, block 64 (seed 1004)."""
    T, H, I, E, k, block = 256, 4096, 14336, 8, 2, 64
    w13, w2, hidden, logits = _moe_problem(1004, T, H, I, E, k)
    d = [dev.htod_sync_copy(v) for v in (to_storage(hidden, DTYPE_BF16), to_storage(logits, DTYPE_BF16), w13, w2)]
    ws_bytes = ops.moe_layer_q4k_workspace_bytes(T, H, I, E, k, block)
    ws, d_out = dev.alloc(ws_bytes), dev.alloc(T * H * 2)
    ops.moe_layer_q4k(d_out, d[0], d[1], d[2], d[3], T, H, I, E, k, block, True, ws, ws_bytes, stream=dev.stream)
    got = fetch(dev, d_out, DTYPE_BF16, (T, H))
    # oracle at full size with f32 BLAS per expert (the f64 loop would take minutes)
    tw, ti = o.topk_softmax(logits, k, True, o.UB_BF16)
    want = np.zeros((T, H), dtype=np.float32)
    parts = np.zeros((T, k, H), dtype=np.float32)
    for e in range(E):
        rows, slots = np.nonzero(ti == e)
        if rows.size == 0:
            continue
        w13d = o.c_dequant(w13.reshape(E, -1)[e], True).reshape(2 * I, H)
        w2d = o.c_dequant(w2.reshape(E, -1)[e], True).reshape(H, I)
        c1 = o.round_through(hidden[rows] @ w13d.T, o.UB_BF16)
        act = o.silu_and_mul(c1, o.UB_BF16)
        parts[rows, slots] = o.round_through((act @ w2d.T) * tw[rows, slots][:, None], o.UB_BF16)
    want = o.topk_sum(parts.reshape(T * k, H), T, k, o.UB_BF16)
    assert o.rel_l2(got, want) < 1e-2
