"""CPU oracle for the quantized-linear + fused-MoE path.  TEST INFRASTRUCTURE ONLY.

Two independent restatements live here:

* numpy functions (this file) written straight from the block-format definitions and
  the scalar reference kernels;
* the C restatement in ``ub_oracle.c`` (built to ``libub_oracle.so`` by the Makefile in
  this folder), reached through :func:`clib`.

Tests cross-check the two against each other, against the ``gguf`` python package and
against the known-answer fixtures.  Only tests, the smoke check and the CPU arm of the
benchmark may import this module; the shipped package never does.

Parity status: PARITY UNPINNED against the reference itself (it holds no golden vectors
for this path and cannot be built without the vendor toolchain).  Dequantisation is
pinned bit-exactly against ``gguf.quants.dequantize`` and hand-computed blocks.

Reference locations (paths inside the reference project):
  formats               kernels/quant.cpp:50-51,98-104,145-150,356-363,392-412
  Q6_K block layout     kernels/quant.cpp:170-177 (declared there, never implemented: the arithmetic is the
                        published GGML one, pinned against the ``gguf`` python package)
  q8_0 quantize         kernels/quant.cpp:270-292
  topk_softmax          kernels/topk_softmax_host.cpp:121-172
  moe_align_block_size  kernels/moe_align_host.cpp:51-58,587-764,766-935
  fused moe GEMM        kernels/fused_moe_host.cpp:43-250
  silu_and_mul          kernels/topsaten_ops_wrapper.cpp:375-391
  weighted combine      kernels/moe_host.cpp:26-81
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

QK8_0 = 32
QK_K = 256
Q8_0_BYTES = 34
Q4K_BYTES = 144
Q6K_BYTES = 210

# dtype codes of the reference's DATATYPE enum (src/lib.rs:87-106)
UB_F16, UB_BF16, UB_F32 = 4, 5, 8

_HERE = os.path.dirname(os.path.abspath(__file__))


# ----------------------------------------------------------------------------- bf16 helpers
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16, returned as uint16 bit patterns."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_through(x: np.ndarray, dtype: int) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    if dtype == UB_F32:
        return x
    if dtype == UB_F16:
        return x.astype(np.float16).astype(np.float32)
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ----------------------------------------------------------------------------- block formats
def pack_q8_0(d_f16: np.ndarray, q: np.ndarray) -> np.ndarray:
    """d_f16 [...,] float16, q [..., 32] int8 -> interleaved bytes [..., 34]."""
    d = np.ascontiguousarray(d_f16, dtype=np.float16)
    q = np.ascontiguousarray(q, dtype=np.int8)
    out = np.empty(d.shape + (Q8_0_BYTES,), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(d.shape + (2,))
    out[..., 2:] = q.view(np.uint8)
    return out


def pack_scales_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Inverse of get_scale_min_k4 (kernels/quant.cpp:356-363): sc, mn [..., 8] in 0..63 -> [..., 12] bytes."""
    sc = np.asarray(sc, dtype=np.uint8)
    mn = np.asarray(mn, dtype=np.uint8)
    out = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    for j in range(4):
        out[..., j] = (sc[..., j] & 63) | ((sc[..., j + 4] >> 4) << 6)
        out[..., j + 4] = (mn[..., j] & 63) | ((mn[..., j + 4] >> 4) << 6)
        out[..., j + 8] = (sc[..., j + 4] & 0xF) | ((mn[..., j + 4] & 0xF) << 4)
    return out


def pack_q4k(d_f16, dmin_f16, sc, mn, q) -> np.ndarray:
    """d, dmin [...] float16; sc, mn [..., 8] in 0..63; q [..., 256] in 0..15 -> bytes [..., 144]."""
    d = np.ascontiguousarray(d_f16, dtype=np.float16)
    dm = np.ascontiguousarray(dmin_f16, dtype=np.float16)
    q = np.asarray(q, dtype=np.uint8).reshape(d.shape + (4, 2, 32))
    out = np.empty(d.shape + (Q4K_BYTES,), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(d.shape + (2,))
    out[..., 2:4] = dm.view(np.uint8).reshape(d.shape + (2,))
    out[..., 4:16] = pack_scales_k4(sc, mn)
    qs = (q[..., 0, :] & 0xF) | (q[..., 1, :] << 4)  # [..., 4, 32]
    out[..., 16:] = qs.reshape(d.shape + (128,))
    return out


def unpack_scales_k4(scales12: np.ndarray):
    s = np.asarray(scales12, dtype=np.uint8)
    sc = np.empty(s.shape[:-1] + (8,), dtype=np.uint8)
    mn = np.empty_like(sc)
    for j in range(4):
        sc[..., j] = s[..., j] & 63
        mn[..., j] = s[..., j + 4] & 63
        sc[..., j + 4] = (s[..., j + 8] & 0xF) | ((s[..., j] >> 6) << 4)
        mn[..., j + 4] = (s[..., j + 8] >> 4) | ((s[..., j + 4] >> 6) << 4)
    return sc, mn


def dequant_q8_0(blocks: np.ndarray) -> np.ndarray:
    """bytes [..., 34] -> f32 [..., 32]; y = d*q."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = b[..., 0:2].copy().view(np.float16).astype(np.float32)  # [..., 1]
    q = b[..., 2:].copy().view(np.int8).astype(np.float32)
    return q * d


def dequant_q4k(blocks: np.ndarray) -> np.ndarray:
    """bytes [..., 144] -> f32 [..., 256]; y = (d*sc)*q - dmin*m."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    lead = b.shape[:-1]
    d = b[..., 0:2].copy().view(np.float16).astype(np.float32)
    dmin = b[..., 2:4].copy().view(np.float16).astype(np.float32)
    sc, mn = unpack_scales_k4(b[..., 4:16])
    dsc = (d * sc.astype(np.float32)).reshape(lead + (4, 2, 1))
    dmn = (dmin * mn.astype(np.float32)).reshape(lead + (4, 2, 1))
    qs = b[..., 16:].reshape(lead + (4, 1, 32))
    q = np.concatenate([qs & 0xF, qs >> 4], axis=-2).astype(np.float32)  # [..., 4, 2, 32]
    return (dsc * q - dmn).reshape(lead + (QK_K,)).astype(np.float32)


def pack_q6k(d_f16: np.ndarray, scales_i8: np.ndarray, q: np.ndarray) -> np.ndarray:
    """d [...] f16, scales [..., 16] int8, q [..., 256] in 0..63 -> bytes [..., 210] = ql[128] qh[64] scales[16] d.
    Value i of a super-block (half h = i // 128, j = (i % 128) // 32, l = i % 32): low nibble in
    ql[64h + 32(j & 1) + l] (high half of the byte when j >= 2), upper two bits at bit 2j of qh[32h + l]."""
    q = np.asarray(q, dtype=np.uint8)
    lead = q.shape[:-1]
    qv = q.reshape(lead + (2, 4, 32))
    ql = np.zeros(lead + (2, 2, 32), dtype=np.uint8)
    qh = np.zeros(lead + (2, 32), dtype=np.uint8)
    for j in range(4):
        ql[..., :, j & 1, :] |= (qv[..., :, j, :] & 0xF) << (4 if j >= 2 else 0)
        qh |= (qv[..., :, j, :] >> 4) << (2 * j)
    d = np.ascontiguousarray(d_f16, dtype=np.float16).reshape(lead + (1,)).view(np.uint8)
    sc = np.ascontiguousarray(scales_i8, dtype=np.int8).view(np.uint8).reshape(lead + (16,))
    return np.concatenate([ql.reshape(lead + (128,)), qh.reshape(lead + (64,)), sc, d], axis=-1)


def dequant_q6k(blocks: np.ndarray) -> np.ndarray:
    """bytes [..., 210] -> f32 [..., 256]; y = (d * scale[i // 16]) * (q - 32), q the 6-bit value."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    lead = b.shape[:-1]
    ql = b[..., 0:128].reshape(lead + (2, 2, 32))
    qh = b[..., 128:192].reshape(lead + (2, 1, 32))
    sc = b[..., 192:208].copy().view(np.int8).astype(np.float32)
    d = b[..., 208:210].copy().view(np.float16).astype(np.float32)
    lo = np.concatenate([ql & 0xF, ql >> 4], axis=-2)  # [..., 2, 4, 32]: j = 0..3
    hi = (qh >> np.array([0, 2, 4, 6], dtype=np.uint8).reshape(4, 1)) & 3
    q = (lo | (hi << 4)).astype(np.int8).astype(np.float32) - np.float32(32)
    dsc = (d * sc).reshape(lead + (16, 1))
    return (dsc * q.reshape(lead + (16, 16))).reshape(lead + (QK_K,)).astype(np.float32)


Q4_0_BYTES = 18
Q5K_BYTES = 176
GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q5_K, GGML_Q6_K = 2, 8, 12, 13, 14  # GGUF type tags


def dequant_q4_0(blocks: np.ndarray) -> np.ndarray:
    """block_q4_0 (kernels/quant.cpp:64-69): f16 d + 16 bytes; value i < 16 is the low nibble of byte i, value
    16 + i its high nibble; y = d * (nibble - 8)."""
    b = np.asarray(blocks, dtype=np.uint8).reshape(-1, Q4_0_BYTES)
    d = b[:, :2].copy().view(np.float16)[:, 0].astype(np.float32)
    q = b[:, 2:]
    lo, hi = (q & 15).astype(np.int32) - 8, (q >> 4).astype(np.int32) - 8
    return (d[:, None] * np.concatenate([lo, hi], axis=1).astype(np.float32)).reshape(-1)


def dequant_q5k(blocks: np.ndarray) -> np.ndarray:
    """block_q5_K (kernels/quant.cpp:154-161): f16 d, f16 dmin, 12 scale bytes (packed as in Q4_K, :356-363),
    qh[32], qs[128].  64-value group g: values 0..31 = low nibbles of qs[32g..] + 16 * bit 2g of qh[l], pair 2g;
    values 32..63 = high nibbles + 16 * bit 2g+1, pair 2g+1; y = (d * sc) * q - dmin * m."""
    b = np.asarray(blocks, dtype=np.uint8).reshape(-1, Q5K_BYTES)
    d = b[:, 0:2].copy().view(np.float16)[:, 0].astype(np.float32)
    dmin = b[:, 2:4].copy().view(np.float16)[:, 0].astype(np.float32)
    sc, mn = unpack_scales_k4(b[:, 4:16])
    qh = b[:, 16:48].astype(np.int32)
    qs = b[:, 48:].reshape(-1, 4, 32).astype(np.int32)
    out = np.empty((b.shape[0], 8, 32), dtype=np.float32)
    for g in range(4):
        q0 = (qs[:, g] & 15) + (((qh >> (2 * g)) & 1) << 4)
        q1 = (qs[:, g] >> 4) + (((qh >> (2 * g + 1)) & 1) << 4)
        out[:, 2 * g] = (d * sc[:, 2 * g].astype(np.float32))[:, None] * q0.astype(np.float32) - (
            dmin * mn[:, 2 * g].astype(np.float32))[:, None]
        out[:, 2 * g + 1] = (d * sc[:, 2 * g + 1].astype(np.float32))[:, None] * q1.astype(np.float32) - (
            dmin * mn[:, 2 * g + 1].astype(np.float32))[:, None]
    return out.reshape(-1)


def dequant_gguf(blob: np.ndarray, ggml_type: int) -> np.ndarray:
    """A GGUF tensor blob (flat bytes of interleaved blocks) of the given GGML type -> flat f32 values."""
    fn, nbytes = {GGML_Q4_0: (dequant_q4_0, Q4_0_BYTES), GGML_Q8_0: (dequant_q8_0, Q8_0_BYTES),
                  GGML_Q4_K: (dequant_q4k, Q4K_BYTES), GGML_Q5_K: (dequant_q5k, Q5K_BYTES),
                  GGML_Q6_K: (dequant_q6k, Q6K_BYTES)}[ggml_type]
    return np.ascontiguousarray(fn(np.asarray(blob, dtype=np.uint8).reshape(-1, nbytes)), dtype=np.float32).reshape(-1)


def gen_q4_0_weight(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    nb = N * K // 32
    b = rng.integers(0, 256, size=(nb, Q4_0_BYTES), dtype=np.uint8)
    b[:, :2] = rng.uniform(1e-3, 1e-2, size=nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    return b.reshape(-1)


def gen_q5k_weight(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    nb = N * K // QK_K
    b = rng.integers(0, 256, size=(nb, Q5K_BYTES), dtype=np.uint8)
    b[:, 0:2] = rng.uniform(1e-4, 1e-2, size=nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    b[:, 2:4] = rng.uniform(1e-4, 1e-2, size=nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    return b.reshape(-1)


def split_layout(inter: np.ndarray, is_q4k: bool) -> np.ndarray:
    """Interleaved GGUF bytes -> the reference's de-interleaved device layout
    (kernels/quant.cpp:219-220, 441-442): all headers first, then all quants."""
    bb = Q4K_BYTES if is_q4k else Q8_0_BYTES
    hb = 16 if is_q4k else 2
    blk = np.ascontiguousarray(inter, dtype=np.uint8).reshape(-1, bb)
    return np.concatenate([blk[:, :hb].reshape(-1), blk[:, hb:].reshape(-1)])


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """f32 [..., 32k] -> bytes [..., k, 34] (kernels/quant.cpp:270-292, roundf rounding)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    xb = x.reshape(x.shape[:-1] + (-1, QK8_0))
    amax = np.abs(xb).max(axis=-1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    v = xb * inv[..., None]
    q = (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.int8)
    return pack_q8_0(d.astype(np.float16), q)


# ----------------------------------------------------------------------------- matmul
def qmatmul_exact(x_f32: np.ndarray, w_deq_f32: np.ndarray) -> np.ndarray:
    """y = x . W^T with float64 accumulation, rounded once to f32."""
    return (x_f32.astype(np.float64) @ w_deq_f32.astype(np.float64).T).astype(np.float32)


def qmatmul_q8act(x_f32: np.ndarray, wq: np.ndarray, N: int, K: int, is_q4k: bool) -> np.ndarray:
    """numpy restatement of the "q8act" arm (see ub_oracle_qmatmul_q8act_f32): activation rows quantised to 8-bit
    blocks, integer block dots, f32 accumulation over blocks in block order."""
    x = np.asarray(x_f32, dtype=np.float32)
    M = x.shape[0]
    if not is_q4k:
        nb = K // QK8_0
        blk = np.asarray(wq, dtype=np.uint8).reshape(N, nb, Q8_0_BYTES)
        dw = blk[..., :2].copy().view(np.float16)[..., 0].astype(np.float32)
        qw = blk[..., 2:].view(np.int8).astype(np.int32)
        xb = x.reshape(M, nb, QK8_0)
        amax = np.abs(xb).max(axis=2)
        d = (amax / np.float32(127.0)).astype(np.float32)
        inv = np.where(d != 0, np.float32(1.0) / np.where(d != 0, d, 1), 0).astype(np.float32)
        v = xb * inv[..., None]
        qx = (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.int32)  # half away from zero
        dx = d.astype(np.float16).astype(np.float32)
        dots = np.einsum("nbi,mbi->mnb", qw, qx).astype(np.float32)
        terms = dots * dw[None] * dx[:, None, :]
    else:
        nb = K // QK_K
        blk = np.asarray(wq, dtype=np.uint8).reshape(N, nb, Q4K_BYTES)
        dw = blk[..., 0:2].copy().view(np.float16)[..., 0].astype(np.float32)
        mw = blk[..., 2:4].copy().view(np.float16)[..., 0].astype(np.float32)
        sc, mn = unpack_scales_k4(blk[..., 4:16])
        qs = blk[..., 16:].reshape(N, nb, 4, 32)
        q4 = np.stack([qs & 0xF, qs >> 4], axis=3).reshape(N, nb, 8, 32).astype(np.int32)
        xb = x.reshape(M, nb, QK_K)
        idx = np.abs(xb).argmax(axis=2)
        mx = np.take_along_axis(xb, idx[..., None], axis=2)[..., 0]
        iscale = np.where(mx != 0, np.float32(-128.0) / np.where(mx != 0, mx, 1), 0).astype(np.float32)
        q8 = np.minimum(np.rint(xb * iscale[..., None]), 127).astype(np.int32).reshape(M, nb, 8, 32)
        dx = np.where(iscale != 0, np.float32(1.0) / np.where(iscale != 0, iscale, 1), 0).astype(np.float32)
        sub = np.einsum("nbji,mbji->mnbj", q4, q8)
        sumi = (sub * sc[None].astype(np.int64)).sum(axis=3).astype(np.float32)
        summ = (q8.sum(axis=3)[:, None] * mn[None].astype(np.int64)).sum(axis=3).astype(np.float32)
        terms = dw[None] * dx[:, None, :] * sumi - mw[None] * dx[:, None, :] * summ
    y = np.zeros((M, N), dtype=np.float32)
    for b in range(terms.shape[2]):
        y += terms[:, :, b]
    return y


def rel_l2(a: np.ndarray, ref: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(a - ref) / (den if den > 0 else 1.0))


# ----------------------------------------------------------------------------- MoE
def topk_softmax(logits_f32: np.ndarray, k: int, norm: bool, dtype: int):
    """kernels/topk_softmax_host.cpp:121-172.  logits already widened to f32 from `dtype`.
    Returns (weights f32 holding values representable in `dtype`, indices int32)."""
    x = np.asarray(logits_f32, dtype=np.float32)
    T, E = x.shape
    mx = x.max(axis=1, keepdims=True)
    ex = np.exp((x - mx).astype(np.float32)).astype(np.float32)
    s = np.zeros((T,), dtype=np.float32)
    for e in range(E):  # same left-to-right f32 summation order as the scalar kernel
        s = (s + ex[:, e]).astype(np.float32)
    inv = np.where(s > 0, np.float32(1.0) / s, np.float32(1.0)).astype(np.float32)
    prob = (ex * inv[:, None]).astype(np.float32)
    w = prob.copy()
    idx = np.zeros((T, k), dtype=np.int32)
    sel = np.zeros((T, k), dtype=np.float32)
    wsum = np.zeros((T,), dtype=np.float32)
    rows = np.arange(T)
    for j in range(k):
        bi = np.argmax(w, axis=1)  # first maximum == strict '>' scan
        idx[:, j] = bi
        p = prob[rows, bi]
        sel[:, j] = round_through(p, dtype)
        wsum = (wsum + p).astype(np.float32)
        w[rows, bi] = -np.inf
    if norm:
        invw = np.where(wsum > 0, np.float32(1.0) / wsum, np.float32(1.0)).astype(np.float32)
        sel = round_through((sel * invw[:, None]).astype(np.float32), dtype)
    return sel, idx


def moe_align_block_size(topk_ids: np.ndarray, E: int, block: int, real_token_num=None, expert_map=None):
    """kernels/moe_align_host.cpp.  Returns (sorted_ids, experts_ids, num_post_pad)."""
    ids = np.asarray(topk_ids, dtype=np.int32)
    T, k = ids.shape
    pad = T * k
    max_padded = T * k + E * (block - 1)
    sorted_ids = np.full((max_padded,), pad, dtype=np.int32)
    experts_ids = np.zeros((max_padded // block,), dtype=np.int32)
    tn = T if real_token_num is None else int(real_token_num)
    flat = ids.reshape(-1)[: tn * k]
    if flat.size == 0:
        return sorted_ids, experts_ids, 0
    if flat.min() < 0 or flat.max() >= E:
        raise ValueError("expert id out of range")
    pos = 0
    blk = 0
    for e in range(E):
        slots = np.nonzero(flat == e)[0].astype(np.int32)  # ascending = stable
        if slots.size == 0:
            continue
        nb = (slots.size + block - 1) // block
        sorted_ids[pos : pos + slots.size] = slots
        experts_ids[blk : blk + nb] = e if expert_map is None else int(expert_map[e])
        pos += nb * block
        blk += nb
    return sorted_ids, experts_ids, pos


def fused_moe(A, B_f32, topk_w, sorted_ids, experts_ids, num_post_pad, top_k, block, mul_routed_weight, dtype,
              C_rows, bias=None, C_init=None):
    """kernels/fused_moe_host.cpp:43-250 with dense f32 expert weights B[E,N,K].
    A is f32 holding values representable in `dtype`.  Returns C [C_rows, N] as f32 values
    rounded through `dtype`; rows no slot names keep C_init (zeros by default)."""
    A = np.asarray(A, dtype=np.float32)
    E, N, K = B_f32.shape
    C = np.zeros((C_rows, N), dtype=np.float32) if C_init is None else np.array(C_init, dtype=np.float32)
    if num_post_pad == 0:
        return C
    topk_ids_size = C_rows
    topk_str = 1 if mul_routed_weight else top_k
    for b in range(num_post_pad // block):
        e = int(experts_ids[b])
        sl = sorted_ids[b * block : (b + 1) * block]
        sl = sl[(sl >= 0) & (sl < topk_ids_size)]
        if sl.size == 0:
            continue
        if e == -1:
            C[sl] = 0.0
            continue
        acc = A[sl // topk_str].astype(np.float64) @ B_f32[e].astype(np.float64).T
        if bias is not None:
            acc = acc + bias[e].astype(np.float64)[None, :]
        if mul_routed_weight:
            acc = acc * np.asarray(topk_w, dtype=np.float32).reshape(-1)[sl].astype(np.float64)[:, None]
        C[sl] = round_through(acc.astype(np.float32), dtype)
    return C


def rms_norm(x_f32: np.ndarray, gamma_f32: np.ndarray, eps: float, dtype: int) -> np.ndarray:
    """RMSNorm as the reference's stand-alone op is used (src/ffi.rs:719-728): the row times rsqrt(mean(x^2) + eps),
    rounded to the storage type, then times gamma, rounded again."""
    x = np.asarray(x_f32, dtype=np.float32)
    ms = (x.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    xn = round_through((x * (1.0 / np.sqrt(ms + eps)).astype(np.float32)).astype(np.float32), dtype)
    return round_through(xn * np.asarray(gamma_f32, dtype=np.float32), dtype)


def silu_and_mul(x_f32: np.ndarray, dtype: int) -> np.ndarray:
    """kernels/topsaten_ops_wrapper.cpp:375-391: out[:, :D] = silu(x[:, :D]) * x[:, D:]."""
    x = np.asarray(x_f32, dtype=np.float32)
    D = x.shape[1] // 2
    g, u = x[:, :D], x[:, D:]
    with np.errstate(over="ignore"):
        s = (g / (np.float32(1.0) + np.exp(-g).astype(np.float32))).astype(np.float32)
    return round_through((s * u).astype(np.float32), dtype)


def topk_sum(x_f32: np.ndarray, T: int, topk: int, dtype: int) -> np.ndarray:
    x = np.asarray(x_f32, dtype=np.float32).reshape(T, topk, -1)
    s = np.zeros((T, x.shape[2]), dtype=np.float32)
    for j in range(topk):
        s = (s + x[:, j]).astype(np.float32)
    return round_through(s, dtype)


def moe_layer_exact(hidden_f32, logits_f32, w13_deq, w2_deq, top_k, block, norm, dtype=UB_BF16,
                    expert_map=None):
    """Whole Mixtral-style layer in the order the reference's caller runs it:
    topk_softmax -> moe_align -> grouped GEMM (w13) -> SiLU*up -> grouped GEMM (w2, routed
    weight) -> sum over top-k.  w13_deq [E, 2I, H] (gate rows first), w2_deq [E, H, I]."""
    T = hidden_f32.shape[0]
    E = w13_deq.shape[0] if expert_map is None else len(expert_map)  # local ids index the local arrays
    tw, ti = topk_softmax(logits_f32, top_k, norm, dtype)
    sorted_ids, experts_ids, npp = moe_align_block_size(ti, E, block, expert_map=expert_map)
    c1 = fused_moe(hidden_f32, w13_deq, None, sorted_ids, experts_ids, npp, top_k, block, 0, dtype, T * top_k)
    act = silu_and_mul(c1, dtype)
    c2 = fused_moe(act, w2_deq, tw, sorted_ids, experts_ids, npp, top_k, block, 1, dtype, T * top_k)
    return topk_sum(c2, T, top_k, dtype), (tw, ti, sorted_ids, experts_ids, npp)


# ----------------------------------------------------------------------------- dense and groupwise W4A16 / W8A16 matmul
def w4a16_dequant(rhs_u8: np.ndarray, scale: np.ndarray, zeros, K: int, N: int, weight_transpose: bool, group_size: int,
                  dtype: int) -> np.ndarray:
    """Enflame W4A16 weights -> dense [K, N] values of `dtype` (kernels/dequant_host.cpp:19-306 is the tiling around a
    vendor unpack routine that is not in the reference tree).  ASSUMED packing, parity unpinned: rhs is [K/2, N]
    ([N, K/2] when transposed); the byte at packed row r holds reduction index 2r in its low nibble and 2r+1 in its
    high nibble; w[k, n] = (q - zeros[k // g, n]) * scale[k // g, n], rounded once to `dtype`."""
    g = group_size if group_size > 0 else K
    rhs = np.asarray(rhs_u8, dtype=np.uint8)
    rhs = rhs.reshape(N, K // 2).T if weight_transpose else rhs.reshape(K // 2, N)
    q = np.empty((K, N), dtype=np.float32)
    q[0::2] = rhs & 15
    q[1::2] = rhs >> 4
    sc = np.repeat(np.asarray(scale, dtype=np.float32).reshape(K // g, N), g, axis=0)
    z = 0.0 if zeros is None else np.repeat(np.asarray(zeros, dtype=np.float32).reshape(K // g, N), g, axis=0)
    return round_through((q - z) * sc, dtype)


def w8a16_dequant(rhs_i8: np.ndarray, scale: np.ndarray, K: int, N: int, rhs_transpose: bool, group_size: int,
                  dtype: int) -> np.ndarray:
    """int8 weights x groupwise scales -> dense [K, N] values of `dtype` (kernels/matmul.cpp:1046-1066)."""
    g = group_size if group_size > 0 else K
    w = np.asarray(rhs_i8, dtype=np.int8)
    w = w.reshape(N, K).T if rhs_transpose else w.reshape(K, N)
    sc = np.repeat(np.asarray(scale, dtype=np.float32).reshape(K // g, N), g, axis=0)
    return round_through(w.astype(np.float32) * sc, dtype)


def dense_matmul(lhs: np.ndarray, rhs: np.ndarray, lhs_transpose: bool, rhs_transpose: bool, dtype: int) -> np.ndarray:
    """out[B, M, N] = lhs[B, M, K] . rhs[B or 1, K, N]; transposed operands are stored [K, M] / [N, K]
    (kernels/matmul.cpp:96-110); accumulation wider than the storage type, one rounding to `dtype` (:480-493)."""
    a = np.asarray(lhs, dtype=np.float64)
    b = np.asarray(rhs, dtype=np.float64)
    if lhs_transpose:
        a = np.swapaxes(a, -1, -2)
    if rhs_transpose:
        b = np.swapaxes(b, -1, -2)
    return round_through((a @ b).astype(np.float32), dtype)


# ----------------------------------------------------------------------------- synthetic inputs
def gen_q8_0_weight(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """int8 quants uniform in [-127,127], f16 scales uniform in [1e-3,1e-2] -> bytes [N, K/32, 34]."""
    q = rng.integers(-127, 128, size=(N, K // QK8_0, QK8_0), dtype=np.int8)
    d = rng.uniform(1e-3, 1e-2, size=(N, K // QK8_0)).astype(np.float16)
    return pack_q8_0(d, q)


def gen_q4k_weight(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """d, dmin f16 uniform in [1e-4,1e-2]; 6-bit scales/mins uniform in [0,63]; nibbles uniform
    in [0,15] -> bytes [N, K/256, 144]."""
    nb = K // QK_K
    d = rng.uniform(1e-4, 1e-2, size=(N, nb)).astype(np.float16)
    dm = rng.uniform(1e-4, 1e-2, size=(N, nb)).astype(np.float16)
    sc = rng.integers(0, 64, size=(N, nb, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(N, nb, 8), dtype=np.uint8)
    q = rng.integers(0, 16, size=(N, nb, QK_K), dtype=np.uint8)
    return pack_q4k(d, dm, sc, mn, q)


def gen_q6k_weight(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """d f16 uniform in [1e-4,1e-3]; int8 scales uniform in [-128,127]; 6-bit quants uniform in [0,63]
    -> bytes [N, K/256, 210]."""
    nb = K // QK_K
    d = rng.uniform(1e-4, 1e-3, size=(N, nb)).astype(np.float16)
    sc = rng.integers(-128, 128, size=(N, nb, 16), dtype=np.int8)
    q = rng.integers(0, 64, size=(N, nb, QK_K), dtype=np.uint8)
    return pack_q6k(d, sc, q)


def gen_activation(rng: np.random.Generator, M: int, K: int, bf16: bool) -> np.ndarray:
    x = rng.standard_normal(size=(M, K), dtype=np.float32)
    return bf16_bits_to_f32(f32_to_bf16_bits(x)) if bf16 else x


# ----------------------------------------------------------------------------- C restatement
_clib = None


def _host_tag() -> str:
    """Short tag of this host's CPU feature flags: the library is built with -march=native,
    so a copy built on another machine must not be loaded."""
    import hashlib

    flags = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = line
                    break
    except OSError:
        pass
    return hashlib.sha1(flags.encode()).hexdigest()[:8]


def build_clib(force: bool = False) -> str:
    name = "libub_oracle_%s.so" % _host_tag()
    so = os.path.join(_HERE, name)
    src = os.path.join(_HERE, "ub_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "OUT=" + name, name])
    return so


def clib() -> ctypes.CDLL:
    """Load (building if needed) the C restatement."""
    global _clib
    if _clib is None:
        h = ctypes.CDLL(build_clib())
        vp, sz, i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        sigs = {
            "ub_oracle_f32_to_f16": [vp, vp, sz], "ub_oracle_f16_to_f32": [vp, vp, sz],
            "ub_oracle_f32_to_bf16": [vp, vp, sz], "ub_oracle_bf16_to_f32": [vp, vp, sz],
            "ub_oracle_dequant_q8_0": [vp, vp, sz], "ub_oracle_dequant_q4k": [vp, vp, sz],
            "ub_oracle_dequant_q6k": [vp, vp, sz],
            "ub_oracle_dequant_to": [vp, vp, sz, i, i],
            "ub_oracle_split_layout": [vp, vp, sz, i], "ub_oracle_interleave_layout": [vp, vp, sz, i],
            "ub_oracle_quantize_q8_0": [vp, vp, sz],
            "ub_oracle_qmatmul_exact": [vp, vp, vp, i, i, i, i], "ub_oracle_qmatmul_f32": [vp, vp, vp, i, i, i, i],
            "ub_oracle_topk_softmax": [vp, vp, vp, i, i, i, i, i],
            "ub_oracle_moe_align": [vp, vp, vp, vp, vp, vp, i, i, i, i],
            "ub_oracle_fused_moe": [vp] * 8 + [i] * 9,
            "ub_oracle_silu_and_mul": [vp, vp, i, i, i], "ub_oracle_topk_sum": [vp, vp, i, i, i, i],
            "ub_oracle_moe_combine": [vp] * 5 + [i] * 5,
            "ub_oracle_indexed_moe": [vp] * 4 + [i] * 7,
            "ub_oracle_qmatmul_q8act_f32": [vp, vp, vp, i, i, i, i],
            "ub_oracle_set_threads": [i],
        }
        for name, args in sigs.items():
            fn = getattr(h, name)
            fn.argtypes = args
            fn.restype = ctypes.c_int if name in ("ub_oracle_moe_align", "ub_oracle_set_threads") else None
        _clib = h
    return _clib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def c_dequant(blocks: np.ndarray, is_q4k: bool) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    bb = Q4K_BYTES if is_q4k else Q8_0_BYTES
    per = QK_K if is_q4k else QK8_0
    nb = b.size // bb
    out = np.empty((nb * per,), dtype=np.float32)
    fn = clib().ub_oracle_dequant_q4k if is_q4k else clib().ub_oracle_dequant_q8_0
    fn(_p(b), _p(out), ctypes.c_size_t(nb))
    return out


# format codes of the C restatement's matmuls (bool is_q4k = 0 / 1)
FMT_Q8_0, FMT_Q4K, FMT_Q6K, FMT_Q5K, FMT_Q4_0 = 0, 1, 2, 3, 4


def c_dequant_q6k(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    nb = b.size // Q6K_BYTES
    out = np.empty((nb * QK_K,), dtype=np.float32)
    clib().ub_oracle_dequant_q6k(_p(b), _p(out), ctypes.c_size_t(nb))
    return out


def c_qmatmul(x_f32: np.ndarray, wq: np.ndarray, N: int, K: int, is_q4k, exact: bool = True) -> np.ndarray:
    """is_q4k: False / True, or one of the FMT_* codes."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    w = np.ascontiguousarray(wq, dtype=np.uint8)
    M = x.shape[0]
    y = np.empty((M, N), dtype=np.float32)
    fn = clib().ub_oracle_qmatmul_exact if exact else clib().ub_oracle_qmatmul_f32
    fn(_p(x), _p(w), _p(y), M, N, K, int(is_q4k))
    return y


def c_qmatmul_q8act(x_f32: np.ndarray, wq: np.ndarray, N: int, K: int, is_q4k) -> np.ndarray:
    """The informational "q8act" arm: activation rows quantised to 8-bit blocks before integer block dots, as
    GGML-family CPU back ends do (Q8_0 blocks against Q8_0 weights, 256-wide int8 blocks against Q4_K weights)."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    w = np.ascontiguousarray(wq, dtype=np.uint8)
    M = x.shape[0]
    y = np.empty((M, N), dtype=np.float32)
    clib().ub_oracle_qmatmul_q8act_f32(_p(x), _p(w), _p(y), M, N, K, int(is_q4k))
    return y


def set_threads(n: int) -> int:
    """Sets the OpenMP thread count of the C restatement; returns the count in effect."""
    return int(clib().ub_oracle_set_threads(int(n)))


def c_quantize_q8_0(x_f32: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    nb = x.size // QK8_0
    out = np.empty((nb, Q8_0_BYTES), dtype=np.uint8)
    clib().ub_oracle_quantize_q8_0(_p(x), _p(out), ctypes.c_size_t(nb))
    return out


def c_topk_softmax(logits_T: np.ndarray, k: int, norm: bool, dtype: int):
    """logits_T: array in the storage type (float32, float16, or uint16 bf16 bits)."""
    a = np.ascontiguousarray(logits_T)
    T, E = a.shape
    w = np.zeros((T, k), dtype=a.dtype)
    idx = np.zeros((T, k), dtype=np.int32)
    clib().ub_oracle_topk_softmax(_p(a), _p(w), _p(idx), T, E, k, int(norm), dtype)
    return w, idx


def c_moe_align(topk_ids: np.ndarray, E: int, block: int, real_token_num=None, expert_map=None):
    ids = np.ascontiguousarray(topk_ids, dtype=np.int32)
    T, k = ids.shape
    max_padded = T * k + E * (block - 1)
    sorted_ids = np.empty((max_padded,), dtype=np.int32)
    experts_ids = np.empty((max_padded // block,), dtype=np.int32)
    npp = np.zeros((1,), dtype=np.int32)
    rt = None if real_token_num is None else np.array([real_token_num], dtype=np.int32)
    em = None if expert_map is None else np.ascontiguousarray(expert_map, dtype=np.int32)
    rc = clib().ub_oracle_moe_align(_p(sorted_ids), _p(experts_ids), _p(npp), _p(ids),
                                    _p(rt) if rt is not None else None, _p(em) if em is not None else None,
                                    E, block, T, k)
    if rc != 0:
        raise ValueError("expert id out of range")
    return sorted_ids, experts_ids, int(npp[0])
