"""GPU parity: GGUF block (de)quantisation through the C-ABI, bit-exact against the oracle."""
import numpy as np
import pytest

import ubridge_b200 as ub
from oracle import oracle as o
from ubridge_b200 import DTYPE_BF16, DTYPE_F16, DTYPE_F32, ops

from _util import ESIZE, NP_STORAGE, fetch, to_storage

pytestmark = pytest.mark.gpu

DTYPES = [DTYPE_F32, DTYPE_F16, DTYPE_BF16]


def _expect(values_f32, dtype):
    return o.round_through(values_f32, {DTYPE_F32: o.UB_F32, DTYPE_F16: o.UB_F16, DTYPE_BF16: o.UB_BF16}[dtype])


def test_golden_blocks(dev, golden):
    for key, is_q4k in (("hand_q8_0", False), ("hand_q4k", True), ("rand_q8_0", False), ("rand_q4k", True)):
        blocks = golden[key + ("_block" if key.startswith("hand") else "_blocks")]
        expect = golden[key + "_expect"]
        d_in = dev.htod_sync_copy(blocks)
        d_out = dev.alloc(expect.size * 4)
        (ops.dequantize_q4k if is_q4k else ops.dequantize_q8_0)(d_out, d_in, expect.size, DTYPE_F32, stream=dev.stream)
        got = dev.dtoh_sync_copy(d_out, np.float32)
        assert np.array_equal(got.view(np.uint32), expect.view(np.uint32)), key


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("is_q4k", [False, True])
@pytest.mark.parametrize("nblocks", [1, 3, 1000, 40001])
def test_dequant_bit_exact(dev, dtype, is_q4k, nblocks):
    rng = np.random.default_rng(nblocks + 17 * is_q4k)
    per = 256 if is_q4k else 32
    w = (o.gen_q4k_weight if is_q4k else o.gen_q8_0_weight)(rng, nblocks, per)
    want = _expect(o.c_dequant(w, is_q4k), dtype)
    d_in = dev.htod_sync_copy(w)
    d_out = dev.alloc(nblocks * per * ESIZE[dtype])
    (ops.dequantize_q4k if is_q4k else ops.dequantize_q8_0)(d_out, d_in, nblocks * per, dtype, stream=dev.stream)
    got = fetch(dev, d_out, dtype, (nblocks * per,))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_full_size_weights(dev):
    """The two benchmark weights, whole: Q8_0 4096x4096 and Q4_K 14336x4096."""
    for seed, is_q4k, N, K in ((1001, False, 4096, 4096), (1002, True, 14336, 4096)):
        rng = np.random.default_rng(seed)
        w = (o.gen_q4k_weight if is_q4k else o.gen_q8_0_weight)(rng, N, K)
        want = o.c_dequant(w, is_q4k)
        d_in = dev.htod_sync_copy(w)
        d_out = dev.alloc(N * K * 4)
        (ops.dequantize_q4k if is_q4k else ops.dequantize_q8_0)(d_out, d_in, N * K, DTYPE_F32, stream=dev.stream)
        got = dev.dtoh_sync_copy(d_out, np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("is_q4k", [False, True])
def test_name_launch_uses_the_split_layout(dev, dtype, is_q4k):
    """get_or_load_func + launch with the reference's kernel names, parameter order and device layout."""
    rng = np.random.default_rng(5)
    nblocks, per = 777, (256 if is_q4k else 32)
    w = (o.gen_q4k_weight if is_q4k else o.gen_q8_0_weight)(rng, nblocks, per)
    split = o.split_layout(w, is_q4k)
    suffix = {DTYPE_F32: "f32", DTYPE_F16: "f16", DTYPE_BF16: "bf16"}[dtype]
    name = "dequantize_block_%s_%s" % ("q4_k" if is_q4k else "q8_0", suffix)
    func = dev.get_or_load_func(name, ub.QUANTIZED)
    d_in = dev.htod_sync_copy(split)
    d_out = dev.alloc(nblocks * per * ESIZE[dtype])
    func.launch(ub.GcuLaunchConfig.for_num_elems(nblocks * per), (d_in, d_out, nblocks * per))
    got = fetch(dev, d_out, dtype, (nblocks * per,))
    want = _expect(o.c_dequant(w, is_q4k), dtype)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # the device-side repack produces the same split bytes
    d_inter = dev.htod_sync_copy(w)
    d_split = dev.alloc(split.size)
    ops.repack_to_split(d_split, d_inter, nblocks, is_q4k, stream=dev.stream)
    assert np.array_equal(dev.dtoh_sync_copy(d_split, np.uint8), split)
    d_back = dev.alloc(split.size)
    ops.repack_to_interleaved(d_back, d_split, nblocks, is_q4k, stream=dev.stream)
    assert np.array_equal(dev.dtoh_sync_copy(d_back, np.uint8), w.reshape(-1))


@pytest.mark.parametrize("dtype", DTYPES)
def test_quantize_q8_0(dev, dtype, golden):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((64, 1024)).astype(np.float32) * 3
    x[0, :32] = 0
    x[1, :64] = golden["quant_q8_0_input"][1]
    xs = to_storage(x, dtype)
    xv = xs.astype(np.float32) if dtype != DTYPE_BF16 else o.bf16_bits_to_f32(xs).reshape(x.shape)
    want = o.c_quantize_q8_0(xv).reshape(-1)
    d_x = dev.htod_sync_copy(xs)
    d_out = dev.alloc(want.size)
    ops.quantize_q8_0(d_out, d_x, x.size, dtype, stream=dev.stream)
    got = dev.dtoh_sync_copy(d_out, np.uint8)
    assert np.array_equal(got, want)
    # name-launch flavour writes the split layout: (T* in, int8* out, in_bytes, out_bytes)
    suffix = {DTYPE_F32: "f32", DTYPE_F16: "f16", DTYPE_BF16: "bf16"}[dtype]
    func = dev.get_or_load_func("quantize_block_q8_0_" + suffix, ub.QUANTIZED)
    d_out2 = dev.alloc(want.size)
    func.launch(ub.GcuLaunchConfig(), (d_x, d_out2, xs.nbytes, want.size))
    assert np.array_equal(dev.dtoh_sync_copy(d_out2, np.uint8), o.split_layout(want, False))


def test_quantize_then_dequantize_roundtrip_bound(dev):
    rng = np.random.default_rng(10)
    x = rng.standard_normal((1 << 16,)).astype(np.float32)
    d_x = dev.htod_sync_copy(x)
    d_q = dev.alloc(x.size // 32 * 34)
    d_y = dev.alloc(x.size * 4)
    ops.quantize_q8_0(d_q, d_x, x.size, DTYPE_F32, stream=dev.stream)
    ops.dequantize_q8_0(d_y, d_q, x.size, DTYPE_F32, stream=dev.stream)
    y = dev.dtoh_sync_copy(d_y, np.float32)
    amax = np.abs(x.reshape(-1, 32)).max(axis=1, keepdims=True)
    # half a quantisation step, plus the f16 rounding of the stored scale (|q| <= 127, 2^-11 relative)
    d = amax / 127
    assert (np.abs(y.reshape(-1, 32) - x.reshape(-1, 32)) <= d * (0.5 + 127 * 2.0 ** -11) * 1.01 + 1e-7).all()
