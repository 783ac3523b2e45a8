"""Generates the known-answer fixtures in this folder.

    python tests/golden/make_golden.py

The reference holds no golden vectors for this path, so these are made from (a) hand-built blocks
whose expected values are written out arithmetically below and (b) the independent ``gguf`` python
package (``gguf.quants.dequantize`` / ``quantize``), which implements the same GGML block formats.
The oracle (``oracle/``) is NOT used to produce expected values here; it is what the fixtures pin.
"""
from __future__ import annotations

import os

import numpy as np
from gguf import GGMLQuantizationType as QT
from gguf import quants

HERE = os.path.dirname(os.path.abspath(__file__))


def f16_bytes(v: float) -> bytes:
    return np.array([v], dtype=np.float16).tobytes()


def hand_q8_0():
    """One block: d = 0.5, q = -16..15  ->  y = q / 2."""
    q = np.arange(-16, 16, dtype=np.int8)
    blk = np.frombuffer(f16_bytes(0.5) + q.tobytes(), dtype=np.uint8).copy()
    expect = q.astype(np.float32) * np.float32(0.5)
    return blk, expect


def hand_q4k():
    """One super-block exercising both halves of the 6-bit packing.
    d = 0.25, dmin = 0.5; scales sc[j] = 1,2,3,4,33,34,35,36 (pairs 4..7 need the two high bits),
    mins m[j] = 0,1,2,3,60,61,62,63; nibble of value i = i % 16."""
    sc = np.array([1, 2, 3, 4, 33, 34, 35, 36], dtype=np.uint8)
    mn = np.array([0, 1, 2, 3, 60, 61, 62, 63], dtype=np.uint8)
    s = np.zeros(12, dtype=np.uint8)
    for j in range(4):
        s[j] = (sc[j] & 63) | ((sc[j + 4] >> 4) << 6)
        s[j + 4] = (mn[j] & 63) | ((mn[j + 4] >> 4) << 6)
        s[j + 8] = (sc[j + 4] & 0xF) | ((mn[j + 4] & 0xF) << 4)
    q = (np.arange(256) % 16).astype(np.uint8)
    qs = np.zeros(128, dtype=np.uint8)
    for g in range(4):
        lo = q[64 * g:64 * g + 32]
        hi = q[64 * g + 32:64 * g + 64]
        qs[32 * g:32 * g + 32] = lo | (hi << 4)
    blk = np.frombuffer(f16_bytes(0.25) + f16_bytes(0.5) + s.tobytes() + qs.tobytes(), dtype=np.uint8).copy()
    expect = np.zeros(256, dtype=np.float32)
    for j in range(8):
        for l in range(32):
            i = 32 * j + l
            expect[i] = np.float32(0.25 * sc[j] * q[i]) - np.float32(0.5 * mn[j])
    return blk, expect


def hand_q6k():
    """One super-block: d = 0.5, scales[k] = k - 8 (both signs), 6-bit value of element i = (5 i + 3) % 64.
    Element i (h = i // 128, j = (i % 128) // 32, l = i % 32): low nibble in ql[64h + 32(j & 1) + l] (upper half
    of the byte for j >= 2), top two bits at bit 2j of qh[32h + l]; y = d * scales[i // 16] * (q - 32)."""
    q = (5 * np.arange(256) + 3) % 64
    sc = (np.arange(16) - 8).astype(np.int8)
    ql = np.zeros(128, dtype=np.uint8)
    qh = np.zeros(64, dtype=np.uint8)
    for i in range(256):
        h, j, l = i // 128, (i % 128) // 32, i % 32
        ql[64 * h + 32 * (j & 1) + l] |= (q[i] & 0xF) << (4 if j >= 2 else 0)
        qh[32 * h + l] |= (q[i] >> 4) << (2 * j)
    blk = np.frombuffer(ql.tobytes() + qh.tobytes() + sc.tobytes() + f16_bytes(0.5), dtype=np.uint8).copy()
    expect = np.array([np.float32(0.5 * sc[i // 16]) * np.float32(q[i] - 32) for i in range(256)], dtype=np.float32)
    return blk, expect


def main() -> None:
    rng = np.random.default_rng(20240601)
    out = {}

    b, e = hand_q8_0()
    out["hand_q8_0_block"], out["hand_q8_0_expect"] = b, e
    assert np.array_equal(quants.dequantize(b, QT.Q8_0).reshape(-1), e)
    b, e = hand_q4k()
    out["hand_q4k_block"], out["hand_q4k_expect"] = b, e
    assert np.array_equal(quants.dequantize(b, QT.Q4_K).reshape(-1), e)

    # random raw bytes are valid blocks of either format as long as the f16 fields are finite
    def random_blocks(n, nbytes, f16_fields):
        raw = rng.integers(0, 256, size=(n, nbytes), dtype=np.uint8)
        for off in f16_fields:
            vals = rng.uniform(-0.05, 0.05, size=n).astype(np.float16)
            raw[:, off:off + 2] = vals.view(np.uint8).reshape(n, 2)
        return raw

    q8 = random_blocks(64, 34, (0,))
    out["rand_q8_0_blocks"] = q8
    out["rand_q8_0_expect"] = quants.dequantize(q8.reshape(-1), QT.Q8_0).reshape(-1).astype(np.float32)
    q4 = random_blocks(24, 144, (0, 2))
    out["rand_q4k_blocks"] = q4
    out["rand_q4k_expect"] = quants.dequantize(q4.reshape(-1), QT.Q4_K).reshape(-1).astype(np.float32)

    # Q8_0 quantisation of a seeded tensor, incl. an all-zero block and exact .5 ties
    x = rng.standard_normal((8, 64)).astype(np.float32)
    x[0, :32] = 0.0
    x[1, :32] = np.arange(32, dtype=np.float32) - 15.5  # amax 16.5: several x*id land near .5
    out["quant_q8_0_input"] = x
    out["quant_q8_0_expect"] = quants.quantize(x, QT.Q8_0).reshape(-1)

    # small matmuls: expected y from gguf-dequantised weights with float64 accumulation
    for name, qt, nb_bytes, N, K in (("mm_q8_0", QT.Q8_0, 34, 24, 256), ("mm_q4k", QT.Q4_K, 144, 24, 512)):
        per = 32 if qt == QT.Q8_0 else 256
        w = random_blocks(N * K // per, nb_bytes, (0,) if qt == QT.Q8_0 else (0, 2))
        xx = rng.standard_normal((5, K)).astype(np.float32)
        wd = quants.dequantize(w.reshape(-1), qt).reshape(N, K).astype(np.float64)
        out[name + "_w"] = w
        out[name + "_x"] = xx
        out[name + "_y"] = (xx.astype(np.float64) @ wd.T).astype(np.float32)

    # Q6_K (drawn after everything above, so the earlier fixtures keep their bytes)
    b, e = hand_q6k()
    out["hand_q6k_block"], out["hand_q6k_expect"] = b, e
    assert np.array_equal(quants.dequantize(b, QT.Q6_K).reshape(-1), e)
    q6 = random_blocks(24, 210, (208,))
    out["rand_q6k_blocks"] = q6
    out["rand_q6k_expect"] = quants.dequantize(q6.reshape(-1), QT.Q6_K).reshape(-1).astype(np.float32)
    N, K = 24, 512
    w = random_blocks(N * K // 256, 210, (208,))
    xx = rng.standard_normal((5, K)).astype(np.float32)
    out["mm_q6k_w"], out["mm_q6k_x"] = w, xx
    out["mm_q6k_y"] = (xx.astype(np.float64) @ quants.dequantize(w.reshape(-1), QT.Q6_K).reshape(N, K)
                       .astype(np.float64).T).astype(np.float32)

    np.savez_compressed(os.path.join(HERE, "blocks.npz"), **out)
    print("wrote", os.path.join(HERE, "blocks.npz"), {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
