"""CPU: the MoE restatements (numpy and C) against vectors PyTorch's own operators produced
(tests/golden/moe_torch.npz, written by tests/golden/make_moe_golden.py)."""
import os

import numpy as np
import pytest

from oracle import oracle as o

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "moe_torch.npz"))
ROUTER = {"mixtral": 2, "wide": 6, "qwen": 8, "all": 4}


@pytest.mark.parametrize("name", sorted(ROUTER))
def test_router_matches_torch_softmax_topk(name):
    k = ROUTER[name]
    logits, idx = G[f"router_{name}_logits"], G[f"router_{name}_idx"]
    for norm, want in ((False, G[f"router_{name}_w"]), (True, G[f"router_{name}_wnorm"])):
        w, i = o.topk_softmax(logits, k, norm, o.UB_F32)
        assert np.array_equal(i, idx)
        assert np.allclose(w, want, rtol=2e-6, atol=1e-9)  # summation order differs: a few f32 ulps
        cw, ci = o.c_topk_softmax(logits, k, norm, o.UB_F32)
        assert np.array_equal(ci, idx)
        assert np.allclose(cw, want, rtol=2e-6, atol=1e-9)


@pytest.mark.parametrize("name", sorted(ROUTER))
@pytest.mark.parametrize("block", [4, 64])
def test_align_matches_torch_stable_argsort(name, block):
    idx = G[f"router_{name}_idx"]
    E = G[f"router_{name}_logits"].shape[1]
    want_s, want_e = G[f"align_{name}_b{block}_sorted"], G[f"align_{name}_b{block}_experts"]
    want_npp = int(G[f"align_{name}_b{block}_npp"][0])
    for fn in (o.moe_align_block_size, o.c_moe_align):
        s, e, npp = fn(idx, E, block)
        assert npp == want_npp
        assert np.array_equal(s, want_s)
        assert np.array_equal(e[: npp // block], want_e[: npp // block])


def test_grouped_gemm_and_combine_match_torch():
    A, B, ids, w = G["gemm_A"], G["gemm_B"], G["gemm_ids"], G["gemm_w"]
    T, k = ids.shape
    E, N, H = B.shape
    for block in (4, 16):
        s, e, npp = o.moe_align_block_size(ids, E, block)
        C = o.fused_moe(A, B, w, s, e, npp, k, block, 0, o.UB_F32, T * k)
        assert np.allclose(C, G["gemm_C"], rtol=1e-6, atol=1e-6)
        # second GEMM's convention: A has one row per slot and the routed weight multiplies the f32 accumulator
        Aslots = A[np.arange(T * k) // k]
        Cw = o.fused_moe(Aslots, B, w, s, e, npp, k, block, 1, o.UB_F32, T * k)
        assert np.allclose(Cw, G["gemm_Cw"], rtol=1e-6, atol=1e-6)
        # C restatement on the same inputs
        Cc = np.zeros((T * k, N), dtype=np.float32)
        o.clib().ub_oracle_fused_moe(o._p(Cc), o._p(np.ascontiguousarray(Aslots)), o._p(B), None, o._p(w), o._p(s),
                                     o._p(e), o._p(np.array([npp], dtype=np.int32)), H, N, E, T * k, k, block, 1, 0,
                                     o.UB_F32)
        assert np.allclose(Cc, G["gemm_Cw"], rtol=1e-6, atol=1e-6)
    # sum over a token's slots (index_add_ in torch)
    y = o.topk_sum(G["gemm_Cw"].astype(np.float32), T, k, o.UB_F32)
    assert np.allclose(y, G["gemm_y"], rtol=1e-5, atol=1e-6)
    # the reference-named combine: y[idx[s]] += e_out[s] * w[idx[s], top[s]]
    yc = np.zeros((T, N), dtype=np.float32)
    e_out = G["gemm_C"].astype(np.float32)
    idx = (np.arange(T * k) // k).astype(np.uint32)
    top = (np.arange(T * k) % k).astype(np.uint32)
    o.clib().ub_oracle_moe_combine(o._p(yc), o._p(e_out), o._p(w), o._p(idx), o._p(top), T, T * k, N, k, o.UB_F32)
    assert np.allclose(yc, G["gemm_y"], rtol=1e-5, atol=1e-6)
