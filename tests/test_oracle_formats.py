"""CPU: the oracle (numpy and C restatements) against the known-answer fixtures and gguf-py."""
import numpy as np
import pytest

from oracle import oracle as o


def test_hand_built_blocks(golden):
    assert np.array_equal(o.dequant_q8_0(golden["hand_q8_0_block"]), golden["hand_q8_0_expect"])
    assert np.array_equal(o.dequant_q4k(golden["hand_q4k_block"]), golden["hand_q4k_expect"])
    assert np.array_equal(o.c_dequant(golden["hand_q8_0_block"], False), golden["hand_q8_0_expect"])
    assert np.array_equal(o.c_dequant(golden["hand_q4k_block"], True), golden["hand_q4k_expect"])


def test_random_blocks_bit_exact(golden):
    for key, is_q4k, fn in (("rand_q8_0", False, o.dequant_q8_0), ("rand_q4k", True, o.dequant_q4k)):
        blocks, expect = golden[key + "_blocks"], golden[key + "_expect"]
        got_np = fn(blocks).reshape(-1)
        got_c = o.c_dequant(blocks, is_q4k)
        assert np.array_equal(got_np.view(np.uint32), expect.view(np.uint32)), key
        assert np.array_equal(got_c.view(np.uint32), expect.view(np.uint32)), key


def test_against_gguf_package_live():
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    rng = np.random.default_rng(7)
    w4 = o.gen_q4k_weight(rng, 16, 1024)
    w8 = o.gen_q8_0_weight(rng, 16, 1024)
    a = quants.dequantize(w4.reshape(-1), gguf.GGMLQuantizationType.Q4_K).reshape(-1).astype(np.float32)
    b = quants.dequantize(w8.reshape(-1), gguf.GGMLQuantizationType.Q8_0).reshape(-1).astype(np.float32)
    assert np.array_equal(o.c_dequant(w4, True).view(np.uint32), a.view(np.uint32))
    assert np.array_equal(o.c_dequant(w8, False).view(np.uint32), b.view(np.uint32))


def test_q6k_against_fixtures_and_gguf_package(golden):
    assert np.array_equal(o.dequant_q6k(golden["hand_q6k_block"]), golden["hand_q6k_expect"])
    got = o.dequant_q6k(golden["rand_q6k_blocks"]).reshape(-1)
    assert np.array_equal(got.view(np.uint32), golden["rand_q6k_expect"].view(np.uint32))
    assert np.array_equal(o.c_dequant_q6k(golden["hand_q6k_block"]), golden["hand_q6k_expect"])
    assert np.array_equal(o.c_dequant_q6k(golden["rand_q6k_blocks"]).view(np.uint32),
                          golden["rand_q6k_expect"].view(np.uint32))
    w = golden["mm_q6k_w"]
    y = o.qmatmul_exact(golden["mm_q6k_x"], o.dequant_q6k(w).reshape(24, 512))
    assert o.rel_l2(y, golden["mm_q6k_y"]) < 1e-6
    assert o.rel_l2(o.c_qmatmul(golden["mm_q6k_x"], w, 24, 512, o.FMT_Q6K), golden["mm_q6k_y"]) < 1e-6
    assert o.rel_l2(o.c_qmatmul(golden["mm_q6k_x"], w, 24, 512, o.FMT_Q6K, exact=False), golden["mm_q6k_y"]) < 1e-5
    # the generator's packing is the inverse of the unpacking
    rng = np.random.default_rng(11)
    d = rng.uniform(1e-3, 1e-2, size=(3, 2)).astype(np.float16)
    sc = rng.integers(-128, 128, size=(3, 2, 16), dtype=np.int8)
    q = rng.integers(0, 64, size=(3, 2, 256), dtype=np.uint8)
    want = (d.astype(np.float32)[..., None] * np.repeat(sc, 16, axis=-1).astype(np.float32)) * \
        (q.astype(np.float32) - np.float32(32))
    assert np.array_equal(o.dequant_q6k(o.pack_q6k(d, sc, q)), want)
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    w6 = o.gen_q6k_weight(rng, 16, 1024)
    a = quants.dequantize(w6.reshape(-1), gguf.GGMLQuantizationType.Q6_K).reshape(-1).astype(np.float32)
    assert np.array_equal(o.dequant_q6k(w6).reshape(-1).view(np.uint32), a.view(np.uint32))


def test_scale_packing_roundtrip():
    rng = np.random.default_rng(3)
    sc = rng.integers(0, 64, size=(100, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(100, 8), dtype=np.uint8)
    s2, m2 = o.unpack_scales_k4(o.pack_scales_k4(sc, mn))
    assert np.array_equal(sc, s2) and np.array_equal(mn, m2)


def test_quantize_q8_0(golden):
    x, expect = golden["quant_q8_0_input"], golden["quant_q8_0_expect"]
    assert np.array_equal(o.quantize_q8_0(x).reshape(-1), expect)
    assert np.array_equal(o.c_quantize_q8_0(x).reshape(-1), expect)


def test_split_layout_roundtrip():
    rng = np.random.default_rng(5)
    for is_q4k, w in ((True, o.gen_q4k_weight(rng, 4, 512)), (False, o.gen_q8_0_weight(rng, 4, 512))):
        split = o.split_layout(w, is_q4k)
        nb = w.size // (144 if is_q4k else 34)
        back = np.empty_like(split)
        o.clib().ub_oracle_interleave_layout(o._p(split), o._p(back), nb, int(is_q4k))
        assert np.array_equal(back, w.reshape(-1))
        again = np.empty_like(split)
        o.clib().ub_oracle_split_layout(o._p(back), o._p(again), nb, int(is_q4k))
        assert np.array_equal(again, split)


def test_matmul_fixtures(golden):
    for name, is_q4k, N, K in (("mm_q8_0", False, 24, 256), ("mm_q4k", True, 24, 512)):
        w, x, y = golden[name + "_w"], golden[name + "_x"], golden[name + "_y"]
        got = o.c_qmatmul(x, w, N, K, is_q4k, exact=True)
        assert np.array_equal(got, y), name  # both are float64 accumulation rounded once
        deq = (o.dequant_q4k if is_q4k else o.dequant_q8_0)(w).reshape(N, K)
        assert np.array_equal(o.qmatmul_exact(x, deq), y)
        fast = o.c_qmatmul(x, w, N, K, is_q4k, exact=False)
        assert o.rel_l2(fast, y) < 1e-5


def test_bf16_helpers():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.14159, 0.0, 65504.0], dtype=np.float32)
    bits = o.f32_to_bf16_bits(x)
    back = o.bf16_bits_to_f32(bits)
    # 1.00390625 = 1 + 2^-8 is a tie and rounds to even (1.0); 1.01171875 = 1 + 3*2^-8 rounds up to 1 + 2^-6
    assert back[0] == 1.0 and back[1] == 1.0 and back[2] == 1.015625
    cb = np.empty_like(bits)
    o.clib().ub_oracle_f32_to_bf16(o._p(x), o._p(cb), x.size)
    assert np.array_equal(cb, bits)
    h = np.empty(x.size, dtype=np.uint16)
    o.clib().ub_oracle_f32_to_f16(o._p(x), o._p(h), x.size)
    assert np.array_equal(h, x.astype(np.float16).view(np.uint16))
    rng = np.random.default_rng(11)
    r = (rng.standard_normal(20000) * np.exp(rng.uniform(-20, 12, 20000))).astype(np.float32)
    h = np.empty(r.size, dtype=np.uint16)
    o.clib().ub_oracle_f32_to_f16(o._p(r), o._p(h), r.size)
    with np.errstate(over="ignore"):
        assert np.array_equal(h, r.astype(np.float16).view(np.uint16))
    f = np.empty(r.size, dtype=np.float32)
    o.clib().ub_oracle_f16_to_f32(o._p(h), o._p(f), r.size)
    assert np.array_equal(f.view(np.uint32), h.view(np.float16).astype(np.float32).view(np.uint32))
