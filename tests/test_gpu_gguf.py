"""GPU parity of the GGUF tensor-blob entries: dispatch on the GGML type tag, Q4_0 and Q5_K dequantisation
(bit-exact against the gguf-py-pinned oracle) and their matmul, and the forwarding of the other tags."""
import os

import numpy as np
import pytest

from oracle import oracle as o
from ubridge_b200 import DTYPE_BF16, DTYPE_F16, DTYPE_F32, ops
from ubridge_b200._lib import UB_ERR_UNSUPPORTED, UbridgeError, lib

from _util import ESIZE, fetch, to_storage

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ODT = {DTYPE_F32: o.UB_F32, DTYPE_F16: o.UB_F16, DTYPE_BF16: o.UB_BF16}
GEN = {o.GGML_Q4_0: o.gen_q4_0_weight, o.GGML_Q8_0: o.gen_q8_0_weight, o.GGML_Q4_K: o.gen_q4k_weight,
       o.GGML_Q5_K: o.gen_q5k_weight, o.GGML_Q6_K: o.gen_q6k_weight}
PER = {o.GGML_Q4_0: 32, o.GGML_Q8_0: 32, o.GGML_Q4_K: 256, o.GGML_Q5_K: 256, o.GGML_Q6_K: 256}


def test_golden_blocks_of_the_two_new_formats(dev):
    more = dict(np.load(os.path.join(ROOT, "tests", "golden", "blocks_more.npz")))
    for key, tag in (("q4_0", o.GGML_Q4_0), ("q5k", o.GGML_Q5_K)):
        blob = more[key].reshape(-1)
        want = more[key + "_f32"]
        d_out = dev.alloc(want.size * 4)
        ops.dequantize_gguf(d_out, dev.htod_sync_copy(blob), tag, want.size, DTYPE_F32, stream=dev.stream)
        got = dev.dtoh_sync_copy(d_out, np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), key


@pytest.mark.parametrize("tag", sorted(GEN))
@pytest.mark.parametrize("dtype", [DTYPE_F32, DTYPE_F16, DTYPE_BF16])
def test_dequant_by_type_tag(dev, tag, dtype):
    rng = np.random.default_rng(tag)
    N, K = 37, 1024
    blob = np.ascontiguousarray(GEN[tag](rng, N, K)).reshape(-1)
    assert lib().ub_gguf_tensor_bytes(tag, N * K) == blob.nbytes
    want = o.round_through(o.dequant_gguf(blob, tag), ODT[dtype])
    d_out = dev.alloc(N * K * ESIZE[dtype])
    ops.dequantize_gguf(d_out, dev.htod_sync_copy(blob), tag, N * K, dtype, stream=dev.stream)
    got = fetch(dev, d_out, dtype, (N * K,))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("tag", sorted(GEN))
@pytest.mark.parametrize("x_dtype", [DTYPE_F32, DTYPE_BF16])
@pytest.mark.parametrize("M,N,K", [(1, 130, 1024), (5, 64, 2048), (11, 33, 512)])
def test_matmul_by_type_tag(dev, tag, x_dtype, M, N, K):
    rng = np.random.default_rng(tag * 100 + M)
    blob = np.ascontiguousarray(GEN[tag](rng, N, K)).reshape(-1)
    x = o.gen_activation(rng, M, K, x_dtype == DTYPE_BF16)
    want = o.qmatmul_exact(x, o.dequant_gguf(blob, tag).reshape(N, K))
    ws_bytes = lib().ub_qmatmul_gguf_workspace_bytes(tag, M, N, K)
    ws = dev.alloc(max(ws_bytes, 256))
    d_y = dev.alloc(M * N * 4)
    ops.qmatmul_gguf(d_y, dev.htod_sync_copy(to_storage(x, x_dtype)), dev.htod_sync_copy(blob), tag, M, N, K,
                     x_dtype=x_dtype, out_dtype=DTYPE_F32, workspace=ws, ws_bytes=ws_bytes, stream=dev.stream)
    got = dev.dtoh_sync_copy(d_y, np.float32, (M, N))
    assert o.rel_l2(got, want) < 1e-3


def test_unknown_type_tag_is_refused(dev):
    d = dev.alloc(4096)
    with pytest.raises(UbridgeError) as ei:
        ops.dequantize_gguf(d, d, 10, 256, DTYPE_F32, stream=dev.stream)  # Q2_K: declared upstream, not taken here
    assert ei.value.status == UB_ERR_UNSUPPORTED
    assert lib().ub_gguf_tensor_bytes(10, 256) == 0
