"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations:
GGUF block-quantized weights packed from random fields, and activations.  Used by ``bench.py`` and by
anything that needs plausible data without a model file; nothing here is a reference implementation.

Block formats as in the reference (kernels/quant.cpp:98-104 ``block_q8_0``, :145-150 ``block_q4_K``,
scale packing :356-363, :170-177 ``block_q6_K``).
"""
from __future__ import annotations

import numpy as np

QK8_0, Q8_0_BYTES = 32, 34
QK_K, Q4K_BYTES = 256, 144
Q6K_BYTES = 210


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 as uint16 (NaN payloads are not preserved)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def pack_q8_0(d_f16: np.ndarray, q: np.ndarray) -> np.ndarray:
    """d [N, nb] f16, q [N, nb, 32] int8 -> bytes [N, nb, 34]."""
    N, nb = d_f16.shape
    out = np.empty((N, nb, Q8_0_BYTES), dtype=np.uint8)
    out[:, :, 0:2] = d_f16.astype(np.float16).view(np.uint8).reshape(N, nb, 2)
    out[:, :, 2:] = q.astype(np.int8).view(np.uint8)
    return out


def pack_q4k(d_f16, dmin_f16, sc, mn, q) -> np.ndarray:
    """d, dmin [N, nb] f16; sc, mn [N, nb, 8] in 0..63; q [N, nb, 256] in 0..15 -> bytes [N, nb, 144]."""
    N, nb = d_f16.shape
    out = np.empty((N, nb, Q4K_BYTES), dtype=np.uint8)
    out[:, :, 0:2] = d_f16.astype(np.float16).view(np.uint8).reshape(N, nb, 2)
    out[:, :, 2:4] = dmin_f16.astype(np.float16).view(np.uint8).reshape(N, nb, 2)
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    # sub-blocks 0..3: six bits in place; 4..7: low nibble in bytes 8..11, top two bits on top of 0..3
    out[:, :, 4:8] = (sc[:, :, 0:4] & 63) | ((sc[:, :, 4:8] >> 4) << 6)
    out[:, :, 8:12] = (mn[:, :, 0:4] & 63) | ((mn[:, :, 4:8] >> 4) << 6)
    out[:, :, 12:16] = (sc[:, :, 4:8] & 15) | ((mn[:, :, 4:8] & 15) << 4)
    # a 64-value group shares 32 bytes: first 32 values in the low nibbles, next 32 in the high ones
    g = q.astype(np.uint8).reshape(N, nb, 4, 2, 32)
    out[:, :, 16:] = (g[:, :, :, 0, :] | (g[:, :, :, 1, :] << 4)).reshape(N, nb, 128)
    return out


def gen_q8_0_weight(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """int8 values uniform in [-127, 127], f16 scales uniform in [1e-3, 1e-2] -> bytes [N, K/32, 34]."""
    nb = K // QK8_0
    q = rng.integers(-127, 128, size=(N, nb, QK8_0), dtype=np.int8)
    d = rng.uniform(1e-3, 1e-2, size=(N, nb)).astype(np.float16)
    return pack_q8_0(d, q)


def gen_q4k_weight(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """d, dmin f16 uniform in [1e-4, 1e-2]; 6-bit scales and mins uniform in [0, 63]; nibbles uniform in
    [0, 15] -> bytes [N, K/256, 144]."""
    nb = K // QK_K
    d = rng.uniform(1e-4, 1e-2, size=(N, nb)).astype(np.float16)
    dm = rng.uniform(1e-4, 1e-2, size=(N, nb)).astype(np.float16)
    sc = rng.integers(0, 64, size=(N, nb, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(N, nb, 8), dtype=np.uint8)
    q = rng.integers(0, 16, size=(N, nb, QK_K), dtype=np.uint8)
    return pack_q4k(d, dm, sc, mn, q)


def gen_q4_0_weight(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """Q4_0: d f16 uniform in [1e-3, 1e-2], every nibble pattern -> bytes [N * K / 32 * 18] (f16 d, sixteen bytes;
    value i in the low nibble of byte i, value 16 + i in its high nibble)."""
    nb = N * K // 32
    b = rng.integers(0, 256, size=(nb, 18), dtype=np.uint8)
    b[:, :2] = rng.uniform(1e-3, 1e-2, size=nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    return b.reshape(-1)


def gen_q5k_weight(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """Q5_K: d, dmin f16 uniform in [1e-4, 1e-2], every pattern of the packed 6-bit scales and mins, the fifth bits
    and the nibbles -> bytes [N * K / 256 * 176] (d, dmin, scales[12], qh[32], qs[128])."""
    nb = N * K // QK_K
    b = rng.integers(0, 256, size=(nb, 176), dtype=np.uint8)
    b[:, 0:2] = rng.uniform(1e-4, 1e-2, size=nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    b[:, 2:4] = rng.uniform(1e-4, 1e-2, size=nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    return b.reshape(-1)


def gen_q6k_weight(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """d f16 uniform in [1e-4, 1e-3]; int8 scales uniform in [-128, 127]; 6-bit quants uniform in [0, 63]
    -> bytes [N, K/256, 210] = ql[128] (low nibbles), qh[64] (upper two bits), scales[16], d.  Position
    128h + 32j + l of a super-block keeps its nibble in ql[64h + 32(j & 1) + l] (upper half of the byte for
    j >= 2) and its top two bits at bit 2j of qh[32h + l]."""
    nb = K // QK_K
    d = rng.uniform(1e-4, 1e-3, size=(N, nb)).astype(np.float16)
    sc = rng.integers(-128, 128, size=(N, nb, 16), dtype=np.int8)
    q = rng.integers(0, 64, size=(N, nb, 2, 4, 32), dtype=np.uint8)
    out = np.zeros((N, nb, Q6K_BYTES), dtype=np.uint8)
    ql = out[:, :, 0:128].reshape(N, nb, 2, 2, 32)
    qh = out[:, :, 128:192].reshape(N, nb, 2, 32)
    for j in range(4):
        ql[:, :, :, j & 1, :] |= (q[:, :, :, j, :] & 0xF) << (4 * (j >> 1))
        qh |= (q[:, :, :, j, :] >> 4) << (2 * j)
    out[:, :, 192:208] = sc.view(np.uint8)
    out[:, :, 208:210] = d.view(np.uint8).reshape(N, nb, 2)
    return out


def gen_activation(rng: np.random.Generator, M: int, K: int, bf16: bool) -> np.ndarray:
    """N(0, 1) activations as f32; with ``bf16`` the values are exactly representable in bf16."""
    x = rng.standard_normal(size=(M, K), dtype=np.float32)
    return bf16_bits_to_f32(f32_to_bf16_bits(x)) if bf16 else x
