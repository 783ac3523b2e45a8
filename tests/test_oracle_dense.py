"""CPU: known answers for the dense / W4A16 / W8A16 restatements (the packing convention is stated in the oracle)."""
import numpy as np

from oracle import oracle as o


def test_w4a16_known_answer():
    rhs = np.array([[0x21, 0x43], [0x65, 0x87]], dtype=np.uint8)          # [K/2 = 2, N = 2]
    scale = np.array([[1.0, 2.0], [0.5, 1.0]], dtype=np.float32)          # group 2 -> [K/g = 2, N]
    zeros = np.array([[1, 0], [0, 8]], dtype=np.float32)
    want = np.array([[0, 6], [1, 8], [2.5, -1], [3, 0]], dtype=np.float32)  # low nibble = even k, high = odd k
    assert np.array_equal(o.w4a16_dequant(rhs, scale, zeros, 4, 2, False, 2, o.UB_F32), want)
    assert np.array_equal(o.w4a16_dequant(rhs.T.copy(), scale, zeros, 4, 2, True, 2, o.UB_F32), want)
    one_group = o.w4a16_dequant(rhs, scale[:1], None, 4, 2, False, -1, o.UB_F32)
    assert np.array_equal(one_group, np.array([[1, 6], [2, 8], [5, 14], [6, 16]], dtype=np.float32))


def test_w8a16_and_dense_known_answer():
    w = np.array([[1, -2], [3, 4], [-128, 127], [0, 5]], dtype=np.int8)    # [K = 4, N = 2]
    scale = np.array([[0.5, 2.0]], dtype=np.float32)
    wd = o.w8a16_dequant(w, scale, 4, 2, False, -1, o.UB_F32)
    assert np.array_equal(wd, w.astype(np.float32) * scale)
    a = np.array([[[1, 2, 0, -1]]], dtype=np.float32)                      # [B = 1, M = 1, K = 4]
    out = o.dense_matmul(a, wd[None], False, False, o.UB_F32)
    assert np.array_equal(out, np.array([[[3.5, 2.0]]], dtype=np.float32))
    out_t = o.dense_matmul(np.swapaxes(a, 1, 2), np.swapaxes(wd[None], 1, 2), True, True, o.UB_F32)
    assert np.array_equal(out_t, out)
