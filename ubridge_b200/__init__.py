"""ubridge_b200: B200 (sm_100a) quantized-linear and fused-MoE path behind Ubridge's operator surface.

All compute lives in ``libubridge_b200.so`` (hand-written CUDA, built in-tree by ``python -m
ubridge_b200.build``); this package is the ctypes binding plus the host-side mirror of the reference's
device / launch / collective types.  Importing the package does not load the library; the first call
does, and raises if it is missing.
"""
from ._lib import (DTYPE_BF16, DTYPE_F16, DTYPE_F32, DTYPE_I32, DTYPE_I8, DTYPE_U8, EXPORTED_SYMBOLS, LIB_PATH,
                   UbridgeError, lib, status_string)
from .device import MATMUL, QUANTIZED, DeviceExecutor, GcuDevice, GcuFunction, GcuLaunchConfig, GcuSlice

__all__ = ["DTYPE_BF16", "DTYPE_F16", "DTYPE_F32", "DTYPE_I32", "DTYPE_I8", "DTYPE_U8", "EXPORTED_SYMBOLS",
           "LIB_PATH", "UbridgeError", "lib", "status_string", "MATMUL", "QUANTIZED", "DeviceExecutor", "GcuDevice",
           "GcuFunction", "GcuLaunchConfig", "GcuSlice"]
