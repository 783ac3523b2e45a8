"""CPU: the informational "q8act" arm (activation rows quantised to 8-bit blocks, integer block dots, the way
GGML-family CPU back ends multiply) - its two restatements agree and its distance to the exact arm is several
times the 1e-3 gate of the decode matmul, so the gate stays on the exact arm."""
import numpy as np
import pytest

from oracle import oracle as o


def test_q8k_style_quantiser_known_answer():
    # one Q4_K row whose weights are all 1 (d = 1, dmin = 0, scales 1, nibbles 1): y = sum(q) / iscale
    K = 256
    w = o.pack_q4k(np.array([[1.0]], np.float16), np.array([[0.0]], np.float16), np.ones((1, 1, 8), np.uint8),
                   np.zeros((1, 1, 8), np.uint8), np.ones((1, 1, 256), np.uint8))
    x = np.zeros((1, K), np.float32)
    x[0, :4] = [-4.0, 2.0, 0.51 / 32, 1.0]          # signed max -4 -> iscale 32: q = -128, 64, round(0.51) = 1, 32
    want = (-128 + 64 + 1 + 32) / 32.0
    assert o.c_qmatmul_q8act(x, w, 1, K, True)[0, 0] == pytest.approx(want, rel=1e-6)
    assert o.qmatmul_q8act(x, w, 1, K, True)[0, 0] == pytest.approx(want, rel=1e-6)


@pytest.mark.parametrize("is_q4k", [False, True])
def test_q8act_restatements_agree_and_differ_from_exact(is_q4k):
    rng = np.random.default_rng(3)
    N, K, M = 96, 2048, 3
    w = (o.gen_q4k_weight if is_q4k else o.gen_q8_0_weight)(rng, N, K)
    x = o.gen_activation(rng, M, K, False)
    a, b = o.c_qmatmul_q8act(x, w, N, K, is_q4k), o.qmatmul_q8act(x, w, N, K, is_q4k)
    assert o.rel_l2(a, b) < 1e-6
    d = o.rel_l2(a, o.c_qmatmul(x, w, N, K, is_q4k))
    assert 1e-3 < d < 3e-2
