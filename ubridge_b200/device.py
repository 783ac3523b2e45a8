"""Host-side mirror of the reference's operator surface, over the C-ABI.

Same names and argument meaning as the Rust types they stand in for:

  GcuDevice        src/gcu_device.rs:61-635   device + one non-blocking stream, alloc / copies / sync
  GcuSlice         src/gcu_slice.rs:49-391    owning device buffer, freed stream-ordered on drop
  GcuFunction      src/gcu_device.rs:160-183, src/gcu_launch.rs:183-328   handle with launch(cfg, params)
  GcuLaunchConfig  src/gcu_launch.rs:40-90
  DeviceExecutor   src/device_executor.rs:57-548  kernel-name tables and has_function / get_function

Differences, on purpose: a missing kernel raises instead of returning a handle whose launch silently
does nothing (src/gcu_device.rs:176-182), and launch errors are reported.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import LaunchConfig, check, lib

QUANTIZED = "quant"   # src/lib.rs:82
MATMUL = "matmul"     # src/lib.rs:78


class GcuLaunchConfig:
    """Grid/block/shared-memory hints.  Accepted for source compatibility; launchers size their own grids."""

    def __init__(self, grid_dim=(1, 1, 1), block_dim=(1, 1, 1), shared_mem_bytes=0, is_cooperative_launch=False):
        self.grid_dim = tuple(grid_dim)
        self.block_dim = tuple(block_dim)
        self.shared_mem_bytes = int(shared_mem_bytes)
        self.is_cooperative_launch = bool(is_cooperative_launch)

    @classmethod
    def for_num_elems(cls, n: int) -> "GcuLaunchConfig":  # src/gcu_launch.rs:63-77
        return cls(grid_dim=((n + 1023) // 1024, 1, 1), block_dim=(1024, 1, 1))

    def as_c(self) -> LaunchConfig:
        c = LaunchConfig()
        c.grid_dim[:] = self.grid_dim
        c.block_dim[:] = self.block_dim
        c.shared_mem_bytes = self.shared_mem_bytes
        c.is_cooperative_launch = int(self.is_cooperative_launch)
        return c


class GcuSlice:
    """Owning device buffer of `nbytes` bytes on `device` (src/gcu_slice.rs:49-101)."""

    def __init__(self, device: "GcuDevice", ptr: int, nbytes: int, owner: Optional["GcuSlice"] = None):
        self.device = device
        self.ptr = ptr or 0
        self.nbytes = nbytes
        self._owner = owner  # sub-views keep their parent alive and never free

    def slice(self, start: int, stop: int) -> "GcuSlice":
        """Byte sub-range view (src/gcu_slice.rs:131-200)."""
        if not (0 <= start <= stop <= self.nbytes):
            raise IndexError("slice out of range")
        return GcuSlice(self.device, self.ptr + start, stop - start, owner=self._owner or self)

    def as_kernel_param(self):
        return ctypes.c_void_p(self.ptr)

    def to_host(self, dtype, shape=None) -> np.ndarray:
        return self.device.dtoh_sync_copy(self, dtype, shape)

    def __del__(self):
        if self._owner is None and self.ptr and self.device is not None and self.device._handle:
            try:
                lib().ub_free(self.device._handle, ctypes.c_void_p(self.ptr))
            except Exception:
                pass
            self.ptr = 0


class GcuFunction:
    """Handle returned by GcuDevice.get_or_load_func; launch(cfg, params) enqueues on the device's stream."""

    def __init__(self, device: "GcuDevice", handle: int, name: str):
        self.device = device
        self._handle = handle
        self.name = name

    @property
    def opcode(self) -> int:
        return lib().ub_function_opcode(self._handle)

    def launch(self, cfg: GcuLaunchConfig, params: Sequence) -> None:
        """params: the kernel's arguments in order; GcuSlice -> device pointer, int -> size_t/int by value."""
        holders = []
        for p in params:
            if isinstance(p, GcuSlice):
                holders.append(ctypes.c_void_p(p.ptr))
            elif isinstance(p, (int, np.integer)):
                holders.append(ctypes.c_size_t(int(p)))
            elif isinstance(p, float):
                holders.append(ctypes.c_float(p))
            else:
                holders.append(p)
        arr = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.pointer(h), ctypes.c_void_p) for h in holders])
        c = cfg.as_c()
        check(lib().ub_launch(self._handle, ctypes.byref(c), arr, self.device.stream), self.name)


class DeviceExecutor:
    """Name tables of the kernels the shim can launch (src/device_executor.rs:119-320, 523-538)."""

    def __init__(self):
        n = lib().ub_function_count()
        self.function_map = {}
        for i in range(n):
            full = lib().ub_function_name(i).decode()
            module, name = full.split("::")
            self.function_map[name] = module

    def has_function(self, module: str, name: str) -> bool:
        return bool(lib().ub_has_function(module.encode(), name.encode()))

    def get_function(self, module: str, name: str) -> int:
        h = lib().ub_get_function(module.encode(), name.encode())
        if not h:
            raise _lib.UbridgeError(_lib.UB_ERR_UNSUPPORTED, "%s::%s" % (module, name))
        return h


class GcuDevice:
    """One device + one non-blocking stream (src/gcu_device.rs:108-139)."""

    def __init__(self, ordinal: int = 0, eager: bool = False):
        h = ctypes.c_void_p()
        check(lib().ub_device_new(ordinal, ctypes.byref(h)), "GcuDevice.new")
        self._handle = h
        self.ordinal = ordinal
        self.is_async = not eager
        self.executor = DeviceExecutor()
        self.stream = ctypes.c_void_p(lib().ub_device_stream(h))

    @staticmethod
    def count() -> int:
        return lib().ub_device_count()

    def bind_to_thread(self) -> None:  # src/gcu_device.rs:144-147
        check(lib().ub_device_bind(self._handle), "bind_to_thread")

    def get_or_load_func(self, func_name: str, module_name: str) -> GcuFunction:
        return GcuFunction(self, self.executor.get_function(module_name, func_name), func_name)

    def has_func(self, func_name: str, module_name: str) -> bool:
        return self.executor.has_function(module_name, func_name)

    # --- memory (src/gcu_device.rs:216-588) ---
    def alloc(self, nbytes: int) -> GcuSlice:
        p = ctypes.c_void_p()
        check(lib().ub_alloc(self._handle, nbytes, ctypes.byref(p)), "alloc")
        return GcuSlice(self, p.value, nbytes)

    def alloc_zeros(self, nbytes: int) -> GcuSlice:
        p = ctypes.c_void_p()
        check(lib().ub_alloc_zeros(self._handle, nbytes, ctypes.byref(p)), "alloc_zeros")
        return GcuSlice(self, p.value, nbytes)

    def htod_copy_into(self, src: np.ndarray, dst: GcuSlice) -> None:
        a = np.ascontiguousarray(src)
        if a.nbytes > dst.nbytes:
            raise ValueError("destination too small")
        check(lib().ub_memcpy_htod(self._handle, ctypes.c_void_p(dst.ptr), a.ctypes.data_as(ctypes.c_void_p), a.nbytes),
              "htod")
        if not a.flags.owndata or a is not src:
            self.synchronize()  # the temporary must outlive the copy

    def htod_sync_copy(self, src: np.ndarray) -> GcuSlice:
        a = np.ascontiguousarray(src)
        s = self.alloc(max(a.nbytes, 1))
        check(lib().ub_memcpy_htod(self._handle, ctypes.c_void_p(s.ptr), a.ctypes.data_as(ctypes.c_void_p), a.nbytes),
              "htod")
        self.synchronize()
        return s

    def dtoh_sync_copy(self, src: GcuSlice, dtype, shape=None) -> np.ndarray:
        dt = np.dtype(dtype)
        n = src.nbytes // dt.itemsize
        out = np.empty((n,), dtype=dt)
        check(lib().ub_memcpy_dtoh(self._handle, out.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(src.ptr),
                                   n * dt.itemsize), "dtoh")
        self.synchronize()
        return out.reshape(shape) if shape is not None else out

    def mem_info(self):
        """(free, total) bytes of device memory."""
        f, t = ctypes.c_size_t(), ctypes.c_size_t()
        check(lib().ub_mem_info(self._handle, ctypes.byref(f), ctypes.byref(t)), "ub_mem_info")
        return f.value, t.value

    def dtod_copy(self, src: GcuSlice, dst: GcuSlice) -> None:
        check(lib().ub_memcpy_dtod(self._handle, ctypes.c_void_p(dst.ptr), ctypes.c_void_p(src.ptr), src.nbytes),
              "dtod")

    def synchronize(self) -> None:
        check(lib().ub_synchronize(self._handle), "synchronize")

    def device_status(self) -> int:
        """Reads and clears the error word kernels set instead of trapping.  Synchronises the stream."""
        return lib().ub_device_status(self.stream)

    def close(self) -> None:
        if self._handle:
            lib().ub_device_free(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
