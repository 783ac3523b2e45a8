"""CPU: the synthetic-input module packs blocks that the oracle unpacks to the fields they were made from."""
import numpy as np

from oracle import oracle as o
from ubridge_b200 import synth


def test_q4k_packing_round_trips_through_the_oracle():
    rng = np.random.default_rng(11)
    N, nb = 5, 3
    d = rng.uniform(1e-4, 1e-2, size=(N, nb)).astype(np.float16)
    dm = rng.uniform(1e-4, 1e-2, size=(N, nb)).astype(np.float16)
    sc = rng.integers(0, 64, size=(N, nb, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(N, nb, 8), dtype=np.uint8)
    q = rng.integers(0, 16, size=(N, nb, 256), dtype=np.uint8)
    blocks = synth.pack_q4k(d, dm, sc, mn, q)
    assert blocks.shape == (N, nb, 144)
    got = o.dequant_q4k(blocks).reshape(N, nb, 8, 32)
    want = (d.astype(np.float32)[..., None, None] * sc.astype(np.float32)[..., None]) * q.reshape(N, nb, 8, 32) \
        - (dm.astype(np.float32)[..., None, None] * mn.astype(np.float32)[..., None])
    assert np.array_equal(got, want.astype(np.float32))


def test_q8_0_packing_round_trips_through_the_oracle():
    rng = np.random.default_rng(12)
    w = synth.gen_q8_0_weight(rng, 4, 128)
    assert w.shape == (4, 4, 34)
    vals = o.dequant_q8_0(w).reshape(4, 4, 32)
    d = w[:, :, :2].copy().view(np.float16).reshape(4, 4).astype(np.float32)
    q = w[:, :, 2:].copy().view(np.int8).astype(np.float32)
    assert np.array_equal(vals, d[..., None] * q)


def test_generators_match_the_oracle_generators_bit_for_bit():
    a = synth.gen_q4k_weight(np.random.default_rng(5), 3, 512)
    b = o.gen_q4k_weight(np.random.default_rng(5), 3, 512)
    assert np.array_equal(a.reshape(-1), b.reshape(-1))
    a8 = synth.gen_q8_0_weight(np.random.default_rng(6), 3, 64)
    b8 = o.gen_q8_0_weight(np.random.default_rng(6), 3, 64)
    assert np.array_equal(a8.reshape(-1), b8.reshape(-1))
    a6 = synth.gen_q6k_weight(np.random.default_rng(8), 3, 512)
    b6 = o.gen_q6k_weight(np.random.default_rng(8), 3, 512)
    assert np.array_equal(a6.reshape(-1), b6.reshape(-1))
    xa = synth.gen_activation(np.random.default_rng(7), 2, 64, True)
    xb = o.gen_activation(np.random.default_rng(7), 2, 64, True)
    assert np.array_equal(xa, xb)
    assert np.array_equal(synth.f32_to_bf16_bits(xa), o.f32_to_bf16_bits(xb))
