"""Generates ``blocks_more.npz``: Q4_0 and Q5_K blocks with the f32 values the independent ``gguf`` python package
(gguf-py) dequantises them to.  Run in an environment that has ``gguf`` installed:

    python tests/golden/make_golden_more.py
"""
import os

import numpy as np
from gguf import GGMLQuantizationType as T
from gguf import quants

HERE = os.path.dirname(os.path.abspath(__file__))
rng = np.random.default_rng(20240613)

q4_0 = rng.integers(0, 256, size=(24, 18), dtype=np.uint8)
q4_0[:, :2] = rng.uniform(1e-3, 1e-1, size=24).astype(np.float16).view(np.uint8).reshape(24, 2)
q4_0[0, 2:] = np.arange(16, dtype=np.uint8) * 17          # nibble pairs (i, i): every code on both halves
q5k = rng.integers(0, 256, size=(12, 176), dtype=np.uint8)
q5k[:, 0:2] = rng.uniform(1e-3, 1e-1, size=12).astype(np.float16).view(np.uint8).reshape(12, 2)
q5k[:, 2:4] = rng.uniform(1e-3, 1e-1, size=12).astype(np.float16).view(np.uint8).reshape(12, 2)
q5k[0, 4:16] = 0xFF                                        # all 6-bit scales and mins at 63
q5k[1, 16:48] = 0xAA                                       # fifth bit set on the odd sub-blocks only

np.savez_compressed(
    os.path.join(HERE, "blocks_more.npz"),
    q4_0=q4_0, q4_0_f32=quants.dequantize(q4_0.reshape(-1), T.Q4_0).astype(np.float32),
    q5k=q5k, q5k_f32=quants.dequantize(q5k.reshape(-1), T.Q5_K).astype(np.float32))
print("wrote blocks_more.npz")
