"""GPU parity of the compatibility entries: name-launched matmul_{f32,f16,bf16}, matmul_{f16,bf16}_{4bit,8bit}
(module "matmul", the reference's 20 / 23 parameter lists) and the dequant_{f16,bf16} export."""
import ctypes

import numpy as np
import pytest

import ubridge_b200 as ub
from oracle import oracle as o
from ubridge_b200 import DTYPE_BF16, DTYPE_F16, DTYPE_F32

from _util import ESIZE, fetch, from_storage, to_storage

pytestmark = pytest.mark.gpu

ODT = {DTYPE_F32: o.UB_F32, DTYPE_F16: o.UB_F16, DTYPE_BF16: o.UB_BF16}
SUFFIX = {DTYPE_F32: "f32", DTYPE_F16: "f16", DTYPE_BF16: "bf16"}
CFG = ub.GcuLaunchConfig()


def _vals(rng, shape, dtype, scale=1.0):
    return from_storage(to_storage((rng.standard_normal(shape) * scale).astype(np.float32), dtype), dtype)


@pytest.mark.parametrize("dtype", [DTYPE_F32, DTYPE_F16, DTYPE_BF16])
@pytest.mark.parametrize("B,M,K,N,lhs_t,rhs_t,bcast", [(1, 1, 64, 40, 0, 0, 1), (3, 65, 100, 67, 0, 0, 0),
                                                       (2, 17, 96, 130, 0, 1, 1), (2, 33, 70, 64, 1, 0, 0),
                                                       (1, 128, 256, 192, 1, 1, 1)])
def test_matmul_by_name(dev, dtype, B, M, K, N, lhs_t, rhs_t, bcast):
    rng = np.random.default_rng(B * 100 + M + N)
    a = _vals(rng, (B, K, M) if lhs_t else (B, M, K), dtype)
    b = _vals(rng, (1 if bcast else B, N, K) if rhs_t else (1 if bcast else B, K, N), dtype, 0.2)
    want = o.dense_matmul(a, b, bool(lhs_t), bool(rhs_t), ODT[dtype])
    func = dev.get_or_load_func("matmul_" + SUFFIX[dtype], ub.MATMUL)
    d_a, d_b = dev.htod_sync_copy(to_storage(a, dtype)), dev.htod_sync_copy(to_storage(b, dtype))
    d_o = dev.alloc(B * M * N * ESIZE[dtype])
    func.launch(CFG, (d_a, d_b, d_o, dtype, B, M, K, N, 1, 1, 0, lhs_t, rhs_t, 1.0, 0.0, 0.0, 32, 64, 64, bcast))
    got = fetch(dev, d_o, dtype, (B, M, N))
    assert o.rel_l2(got, want) < (1e-5 if dtype == DTYPE_F32 else 3e-3)


@pytest.mark.parametrize("dtype", [DTYPE_F16, DTYPE_BF16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,K,N,group,rhs_t", [(1, 256, 96, 128, 0), (5, 512, 130, 64, 0), (40, 256, 64, -1, 0),
                                               (3, 384, 72, 128, 1)])
def test_groupwise_matmul_by_name(dev, dtype, bits, M, K, N, group, rhs_t):
    rng = np.random.default_rng(M + K + N + bits)
    g = group if group > 0 else K
    a = _vals(rng, (1, M, K), dtype)
    scale = from_storage(to_storage(rng.uniform(0.01, 0.05, size=(K // g, N)).astype(np.float32), dtype), dtype)
    if bits == 4:
        rhs = rng.integers(0, 256, size=(N, K // 2) if rhs_t else (K // 2, N), dtype=np.uint8)
        zeros = from_storage(to_storage(rng.integers(0, 16, size=(K // g, N)).astype(np.float32), dtype), dtype)
        wd = o.w4a16_dequant(rhs, scale, zeros, K, N, bool(rhs_t), group, ODT[dtype])
        d_z = dev.htod_sync_copy(to_storage(zeros, dtype))
    else:
        rhs = rng.integers(-128, 128, size=(N, K) if rhs_t else (K, N), dtype=np.int8)
        wd = o.w8a16_dequant(rhs, scale, K, N, bool(rhs_t), group, ODT[dtype])
        d_z = dev.alloc(256)  # the 8-bit kernel takes the pointer and ignores it
    want = o.dense_matmul(a, wd[None], False, False, ODT[dtype])
    func = dev.get_or_load_func("matmul_%s_%dbit" % (SUFFIX[dtype], bits), ub.MATMUL)
    d_a, d_b = dev.htod_sync_copy(to_storage(a, dtype)), dev.htod_sync_copy(rhs)
    d_s = dev.htod_sync_copy(to_storage(scale, dtype))
    d_o = dev.alloc(M * N * 2)
    func.launch(CFG, (d_a, d_b, d_o, d_s, d_z, dtype, 1, M, K, N, 1, 1, 0, 0, rhs_t, 1.0, 0.0, 0.0, 32, 64, 64, 1,
                      group))
    got = fetch(dev, d_o, dtype, (1, M, N))
    assert o.rel_l2(got, want) < 3e-3  # one rounding to the 16-bit output type


@pytest.mark.parametrize("dtype", [DTYPE_F16, DTYPE_BF16])
@pytest.mark.parametrize("K,N,group,transpose", [(256, 96, 128, 0), (128, 130, -1, 0), (512, 33, 64, 1)])
def test_dequant_export(dev, dtype, K, N, group, transpose):
    rng = np.random.default_rng(K + N)
    g = group if group > 0 else K
    rhs = rng.integers(0, 256, size=(N, K // 2) if transpose else (K // 2, N), dtype=np.uint8)
    scale = from_storage(to_storage(rng.uniform(0.01, 0.05, size=(K // g, N)).astype(np.float32), dtype), dtype)
    zeros = from_storage(to_storage(rng.integers(0, 16, size=(K // g, N)).astype(np.float32), dtype), dtype)
    want = o.w4a16_dequant(rhs, scale, zeros, K, N, bool(transpose), group, ODT[dtype])
    d_r, d_s, d_z = dev.htod_sync_copy(rhs), dev.htod_sync_copy(to_storage(scale, dtype)), dev.htod_sync_copy(
        to_storage(zeros, dtype))
    d_o = dev.alloc(K * N * 2)
    fn = getattr(ub.lib(), "dequant_" + SUFFIX[dtype])
    fn(ctypes.c_void_p(d_o.ptr), ctypes.c_void_p(d_r.ptr), ctypes.c_void_p(d_s.ptr), ctypes.c_void_p(d_z.ptr), K, N,
       transpose, group, dev.stream)
    assert ub.lib().ub_last_status() == 0
    got = fetch(dev, d_o, dtype, (K, N))
    assert np.array_equal(got, want)  # (q - z) * s is exact in f32 before the one rounding
