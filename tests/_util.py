"""Helpers shared by the GPU parity tests: host<->device staging in the storage types."""
import numpy as np

from oracle import oracle as o
from ubridge_b200 import DTYPE_BF16, DTYPE_F16, DTYPE_F32

NP_STORAGE = {DTYPE_F32: np.float32, DTYPE_F16: np.float16, DTYPE_BF16: np.uint16}
ESIZE = {DTYPE_F32: 4, DTYPE_F16: 2, DTYPE_BF16: 2}


def to_storage(x_f32: np.ndarray, dtype: int) -> np.ndarray:
    """f32 values -> host array in the storage type (bf16 as uint16 bit patterns)."""
    if dtype == DTYPE_F32:
        return np.ascontiguousarray(x_f32, dtype=np.float32)
    if dtype == DTYPE_F16:
        return np.ascontiguousarray(x_f32).astype(np.float16)
    return o.f32_to_bf16_bits(x_f32).reshape(np.shape(x_f32))


def from_storage(a: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == DTYPE_F32:
        return a.astype(np.float32)
    if dtype == DTYPE_F16:
        return a.astype(np.float32)
    return o.bf16_bits_to_f32(a).reshape(a.shape)


def fetch(dev, buf, dtype: int, shape) -> np.ndarray:
    """Device buffer in storage type -> f32 values on the host."""
    n = int(np.prod(shape))
    raw = dev.dtoh_sync_copy(buf.slice(0, n * ESIZE[dtype]), NP_STORAGE[dtype], shape)
    return from_storage(raw, dtype)
