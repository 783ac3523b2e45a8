"""CPU: known-answer cases for the MoE router, alignment, grouped GEMM and combine restatements."""
import ctypes

import numpy as np
import pytest

from oracle import oracle as o


def test_topk_softmax_ties_go_to_lowest_index():
    logits = np.array([[1.0, 3.0, 3.0, 0.0], [2.0, 2.0, 2.0, 2.0]], dtype=np.float32)
    w, idx = o.topk_softmax(logits, 2, False, o.UB_F32)
    assert idx.tolist() == [[1, 2], [0, 1]]
    assert np.allclose(w[1], [0.25, 0.25])
    cw, cidx = o.c_topk_softmax(logits, 2, False, o.UB_F32)
    assert np.array_equal(cidx, idx) and np.allclose(cw, w, atol=1e-7)


def test_topk_softmax_norm_and_storage_rounding():
    logits = np.array([[0.0, np.log(3.0), -50.0]], dtype=np.float32)  # probs ~ 0.25, 0.75, 0
    for norm in (False, True):
        w, idx = o.topk_softmax(logits, 2, norm, o.UB_F32)
        assert idx.tolist() == [[1, 0]]
        assert np.allclose(w, [[0.75, 0.25]], atol=1e-6)
    # bf16 storage: weight is rounded to bf16 BEFORE the renormalisation and once more after it
    lg = o.bf16_bits_to_f32(o.f32_to_bf16_bits(np.array([[0.3, -1.2, 0.9, 0.1]], dtype=np.float32)))
    w, idx = o.topk_softmax(lg, 2, True, o.UB_BF16)
    p = np.exp(lg - lg.max())
    p = p / p.sum()
    sel = o.round_through(p[0, idx[0]], o.UB_BF16)
    want = o.round_through(sel * (np.float32(1.0) / (p[0, idx[0]].sum(dtype=np.float32))), o.UB_BF16)
    assert np.allclose(w[0], want, rtol=2 ** -7)
    cw, cidx = o.c_topk_softmax(o.f32_to_bf16_bits(lg), 2, True, o.UB_BF16)
    assert np.array_equal(cidx, idx)
    assert np.array_equal(o.bf16_bits_to_f32(cw), w)


ALIGN_CASES = {
    # ids [T,k], E, block -> sorted_ids, experts_ids, num_post_pad    (pad value = T*k)
    "empty_expert": (np.array([[0, 2], [2, 0], [2, 2]]), 3, 2,
                     [0, 3, 1, 2, 4, 5, 6, 6, 6], [0, 2, 2, 0], 6),
    "exact_block": (np.array([[1], [1], [0], [1], [1]]), 2, 4,
                    [2, 5, 5, 5, 0, 1, 3, 4, 5, 5, 5], [0, 1], 8),
    "all_to_one": (np.array([[1, 1], [1, 1]]), 2, 3,
                   [0, 1, 2, 3, 4, 4, 4, 4], [1, 1], 6),
}


@pytest.mark.parametrize("name", sorted(ALIGN_CASES))
def test_moe_align_known_answers(name):
    ids, E, block, want_sorted, want_experts, want_npp = ALIGN_CASES[name]
    for fn in (o.moe_align_block_size, o.c_moe_align):
        s, e, npp = fn(ids.astype(np.int32), E, block)
        assert s.tolist() == want_sorted, (name, fn.__name__)
        assert e.tolist() == want_experts + [0] * (len(e) - len(want_experts)) or e.tolist() == want_experts
        assert npp == want_npp


def test_moe_align_expert_map_and_real_token_num():
    ids = np.array([[0, 1], [1, 2], [2, 0], [3, 3]], dtype=np.int32)
    emap = np.array([-1, 0, 1, -1], dtype=np.int32)
    for fn in (o.moe_align_block_size, o.c_moe_align):
        s, e, npp = fn(ids, 4, 2, expert_map=emap)
        # experts 0..3 hold slots {0,5}, {1,2}, {3,4}, {6,7}; ids are replaced by the map entry
        assert s[:8].tolist() == [0, 5, 1, 2, 3, 4, 6, 7] and npp == 8
        assert e[:4].tolist() == [-1, 0, 1, -1]
        s, e, npp = fn(ids, 4, 2, real_token_num=2)
        # only slots 0..3 are read: expert 0 {0}, expert 1 {1,2}, expert 2 {3}; pad value stays T*k = 8
        assert s[:6].tolist() == [0, 8, 1, 2, 3, 8] and npp == 6
        assert e[:3].tolist() == [0, 1, 2]
        s, e, npp = fn(ids, 4, 2, real_token_num=0)
        assert npp == 0 and (s == 8).all() and (e == 0).all()


def test_moe_align_rejects_bad_ids():
    with pytest.raises(ValueError):
        o.c_moe_align(np.array([[0, 5]], dtype=np.int32), 4, 2)
    with pytest.raises(ValueError):
        o.moe_align_block_size(np.array([[0, -1]], dtype=np.int32), 4, 2)


def _rand_moe(rng, T, H, N, E, k):
    A = o.bf16_bits_to_f32(o.f32_to_bf16_bits(rng.standard_normal((T, H)).astype(np.float32)))
    B = o.bf16_bits_to_f32(o.f32_to_bf16_bits((rng.standard_normal((E, N, H)) * 0.1).astype(np.float32)))
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    w = rng.uniform(0.1, 1.0, size=(T, k)).astype(np.float32)
    return A, B, ids, w


def test_fused_moe_numpy_vs_c():
    rng = np.random.default_rng(21)
    T, H, N, E, k, block = 9, 32, 12, 4, 2, 4
    A, B, ids, w = _rand_moe(rng, T, H, N, E, k)
    s, e, npp = o.moe_align_block_size(ids, E, block)
    for mul in (0, 1):
        Ain = A if not mul else o.bf16_bits_to_f32(o.f32_to_bf16_bits(rng.standard_normal((T * k, H)).astype(np.float32)))
        want = o.fused_moe(Ain, B, w, s, e, npp, k, block, mul, o.UB_BF16, T * k)
        C = np.zeros((T * k, N), dtype=np.uint16)
        Ab = o.f32_to_bf16_bits(Ain)
        npp_arr = np.array([npp], dtype=np.int32)
        o.clib().ub_oracle_fused_moe(o._p(C), o._p(Ab), o._p(B), None, o._p(w),
                                     o._p(s), o._p(e), o._p(npp_arr), H, N, E, T * k, k, block, mul,
                                     0, o.UB_BF16)
        assert np.array_equal(o.bf16_bits_to_f32(C), want)
    # direct definition: every slot row equals the token row times its expert
    want = o.fused_moe(A, B, w, s, e, npp, k, block, 0, o.UB_F32, T * k)
    for slot in range(T * k):
        ref = A[slot // k].astype(np.float64) @ B[ids.reshape(-1)[slot]].astype(np.float64).T
        assert np.allclose(want[slot], ref, rtol=1e-6, atol=1e-6)


def test_fused_moe_expert_minus_one_zero_fills():
    rng = np.random.default_rng(22)
    T, H, N, E, k, block = 6, 16, 8, 4, 2, 4
    A, B, ids, w = _rand_moe(rng, T, H, N, E, k)
    emap = np.array([0, -1, 1, -1], dtype=np.int32)
    s, e, npp = o.moe_align_block_size(ids, E, block, expert_map=emap)
    C0 = np.full((T * k, N), 7.0, dtype=np.float32)
    C = o.fused_moe(A, B[[0, 2]], w, s, e, npp, k, block, 0, o.UB_F32, T * k, C_init=C0)
    flat = ids.reshape(-1)
    for slot in range(T * k):
        if emap[flat[slot]] == -1:
            assert (C[slot] == 0).all()
        else:
            assert not (C[slot] == 7.0).any()


def test_silu_sum_combine():
    rng = np.random.default_rng(23)
    x = rng.standard_normal((5, 8)).astype(np.float32)
    want = o.silu_and_mul(x, o.UB_F32)
    out = np.zeros((5, 4), dtype=np.float32)
    o.clib().ub_oracle_silu_and_mul(o._p(x), o._p(out), 5, 4, o.UB_F32)
    assert np.allclose(out, want, rtol=1e-6)
    g, u = x[:, :4], x[:, 4:]
    assert np.allclose(want, g / (1 + np.exp(-g)) * u, rtol=1e-6)
    # weighted combine, applied in ascending k with storage rounding at both steps
    N, K, M, topk = 3, 5, 4, 2
    y = np.zeros((N, M), dtype=np.float16)
    e_out = rng.standard_normal((K, M)).astype(np.float16)
    w = rng.uniform(0, 1, size=(N, topk)).astype(np.float32)
    idx = np.array([0, 2, 0, 7, 1], dtype=np.uint32)   # 7 is out of range: skipped
    top = np.array([0, 1, 1, 0, 5], dtype=np.uint32)   # 5 >= topk: skipped
    o.clib().ub_oracle_moe_combine(o._p(y), o._p(e_out), o._p(w), o._p(idx), o._p(top),
                                   N, K, M, topk, o.UB_F16)
    want = np.zeros((N, M), dtype=np.float16)
    for k in (0, 1, 2):
        r = int(idx[k])
        prod = (e_out[k].astype(np.float32) * w[r, top[k]]).astype(np.float16)
        want[r] = (want[r].astype(np.float32) + prod.astype(np.float32)).astype(np.float16)
    assert np.array_equal(y, want)


def test_moe_layer_matches_direct_definition():
    rng = np.random.default_rng(24)
    T, H, I, E, k, block = 7, 256, 256, 4, 2, 4
    hidden = o.gen_activation(rng, T, H, True)
    logits = o.gen_activation(rng, T, E, True)
    w13 = o.dequant_q4k(o.gen_q4k_weight(rng, E * 2 * I, H)).reshape(E, 2 * I, H)
    w2 = o.dequant_q4k(o.gen_q4k_weight(rng, E * H, I)).reshape(E, H, I)
    out, (tw, ti, *_rest) = o.moe_layer_exact(hidden, logits, w13, w2, k, block, True)
    ref = np.zeros((T, H), dtype=np.float64)
    for t in range(T):
        for j in range(k):
            e = ti[t, j]
            gu = w13[e].astype(np.float64) @ hidden[t].astype(np.float64)
            g, u = gu[:I], gu[I:]
            act = g / (1 + np.exp(-g)) * u
            ref[t] += tw[t, j] * (w2[e].astype(np.float64) @ act)
    assert o.rel_l2(out, ref) < 2e-2  # the layer rounds to bf16 at four points; the direct sum does not
