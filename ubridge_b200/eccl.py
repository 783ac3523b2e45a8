"""Collectives with the reference's eccl surface (src/eccl.rs:14-426) over the NCCL-backed C-ABI.

``Id`` is the 128-byte unique id shipped out of band (src/eccl.rs:24-43); ``Comm.from_rank`` is one rank
per process or thread (src/eccl.rs:181-206); every collective enqueues on the stream given (the
device's single stream in the reference, src/eccl.rs:209-413).
"""
from __future__ import annotations

import ctypes
import time

from . import _lib
from ._lib import EcclUniqueId, lib


class EcclError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__("eccl: %s failed with result %d" % (what, code))
        self.code = code


class EcclTimeout(EcclError):
    """A collective did not complete within the host's deadline; the communicator has been aborted."""

    def __init__(self, what: str, seconds: float):
        RuntimeError.__init__(self, "eccl: %s did not complete within %.3f s; communicator aborted" % (what, seconds))
        self.code = 6  # UB_ERR_TIMEOUT


class ReduceOp:
    Sum, Prod, Max, Min, Avg = 0, 1, 2, 3, 4  # src/eccl.rs:45-61


# ecclDataType_t (src/eccl.rs:86-96)
Int8, Uint8, Int32, Uint32, Int64, Uint64, Float16, Float32, Float64, Bfloat16 = range(10)

_FROM_UB_DTYPE = {_lib.DTYPE_F32: Float32, _lib.DTYPE_F16: Float16, _lib.DTYPE_BF16: Bfloat16,
                  _lib.DTYPE_I32: Int32, _lib.DTYPE_I8: Int8, _lib.DTYPE_U8: Uint8}


def eccl_dtype(ub_dtype: int) -> int:
    return _FROM_UB_DTYPE[ub_dtype]


def _ok(rc: int, what: str) -> None:
    if rc != 0:
        raise EcclError(rc, what)


def _p(buf):
    if buf is None:
        return None
    if hasattr(buf, "ptr"):
        return ctypes.c_void_p(buf.ptr)
    if isinstance(buf, ctypes.c_void_p):
        return buf
    return ctypes.c_void_p(int(buf))


def get_version() -> int:
    v = ctypes.c_int()
    _ok(lib().ecclGetVersion(ctypes.byref(v)), "ecclGetVersion")
    return v.value


class Id:
    def __init__(self, raw: bytes | None = None):
        self._id = EcclUniqueId()
        if raw is None:
            _ok(lib().ecclGetUniqueId(ctypes.byref(self._id)), "ecclGetUniqueId")
        else:
            if len(raw) != 128:
                raise ValueError("unique id is 128 bytes")
            ctypes.memmove(ctypes.byref(self._id), raw, 128)

    @classmethod
    def uninit(cls, internal: bytes) -> "Id":  # src/eccl.rs:35-38
        return cls(internal)

    def internal(self) -> bytes:
        return ctypes.string_at(ctypes.byref(self._id), 128)


def group_start() -> None:
    _ok(lib().ecclGroupStart(), "ecclGroupStart")


def group_end() -> None:
    _ok(lib().ecclGroupEnd(), "ecclGroupEnd")


class Comm:
    def __init__(self, handle, rank: int, world_size: int):
        self._comm = handle
        self.rank = rank
        self.world_size = world_size

    @classmethod
    def from_rank(cls, rank: int, world_size: int, uid: Id) -> "Comm":
        """The calling thread's current CUDA device becomes this rank's device."""
        h = ctypes.c_void_p()
        _ok(lib().ecclCommInitRank(ctypes.byref(h), world_size, uid._id, rank), "ecclCommInitRank")
        return cls(h, rank, world_size)

    @classmethod
    def from_devices(cls, ordinals) -> list["Comm"]:  # src/eccl.rs:120-141
        n = len(ordinals)
        arr = (ctypes.c_void_p * n)()
        devs = (ctypes.c_int * n)(*ordinals)
        _ok(lib().ecclCommInitAll(arr, n, devs), "ecclCommInitAll")
        return [cls(ctypes.c_void_p(arr[i]), i, n) for i in range(n)]

    def count(self) -> int:
        v = ctypes.c_int()
        _ok(lib().ecclCommCount(self._comm, ctypes.byref(v)), "ecclCommCount")
        return v.value

    def device(self) -> int:
        v = ctypes.c_int()
        _ok(lib().ecclCommDevice(self._comm, ctypes.byref(v)), "ecclCommDevice")
        return v.value

    def user_rank(self) -> int:
        v = ctypes.c_int()
        _ok(lib().ecclCommUserRank(self._comm, ctypes.byref(v)), "ecclCommUserRank")
        return v.value

    def all_reduce(self, send, recv, count: int, dtype: int, op: int = ReduceOp.Sum, stream=None) -> None:
        _ok(lib().ecclAllReduce(_p(send), _p(recv), count, dtype, op, self._comm, _p(stream)), "ecclAllReduce")

    def reduce(self, send, recv, count: int, dtype: int, op: int, root: int, stream=None) -> None:
        _ok(lib().ecclReduce(_p(send), _p(recv), count, dtype, op, root, self._comm, _p(stream)), "ecclReduce")

    def broadcast(self, send, recv, count: int, dtype: int, root: int, stream=None) -> None:
        _ok(lib().ecclBroadcast(_p(send), _p(recv), count, dtype, root, self._comm, _p(stream)), "ecclBroadcast")

    def all_gather(self, send, recv, sendcount: int, dtype: int, stream=None) -> None:
        _ok(lib().ecclAllGather(_p(send), _p(recv), sendcount, dtype, self._comm, _p(stream)), "ecclAllGather")

    def reduce_scatter(self, send, recv, recvcount: int, dtype: int, op: int = ReduceOp.Sum, stream=None) -> None:
        _ok(lib().ecclReduceScatter(_p(send), _p(recv), recvcount, dtype, op, self._comm, _p(stream)),
            "ecclReduceScatter")

    def send(self, buf, count: int, dtype: int, peer: int, stream=None) -> None:
        _ok(lib().ecclSend(_p(buf), count, dtype, peer, self._comm, _p(stream)), "ecclSend")

    def recv(self, buf, count: int, dtype: int, peer: int, stream=None) -> None:
        _ok(lib().ecclRecv(_p(buf), count, dtype, peer, self._comm, _p(stream)), "ecclRecv")

    def async_error(self) -> int:
        """ncclCommGetAsyncError: 0 while the communicator is healthy."""
        v = ctypes.c_int()
        _ok(lib().ub_eccl_comm_async_error(self._comm, ctypes.byref(v)), "ub_eccl_comm_async_error")
        return v.value

    def wait(self, stream, timeout_s: float, poll_s: float = 0.0005, what: str = "collective", query=None,
             clock=time.monotonic, sleep=time.sleep) -> None:
        """Bound the work enqueued on `stream` (collectives of this communicator among it) by a host deadline:
        poll the stream and the communicator's asynchronous error state; on an error or on expiry abort the
        communicator (what the reference's Drop does, src/eccl.rs:63-70) and raise, so that the caller is never
        left blocking on a peer that has gone away.  `query` returns UB_OK / UB_ERR_NOT_READY / an error code
        (default: ub_stream_query on `stream`)."""
        if query is None:
            query = lambda: lib().ub_stream_query(_p(stream))  # noqa: E731
        deadline = clock() + timeout_s
        while True:
            st = query()
            if st == _lib.UB_OK:
                return
            if st != _lib.UB_ERR_NOT_READY:
                self.abort()
                raise EcclError(st, what + " (stream)")
            err = self.async_error()
            if err not in (0, 7):  # ecclSuccess, ecclInProgress
                self.abort()
                raise EcclError(err, what + " (asynchronous error)")
            if clock() >= deadline:
                self.abort()
                raise EcclTimeout(what, timeout_s)
            sleep(poll_s)

    def destroy(self) -> None:
        if self._comm:
            lib().ecclCommDestroy(self._comm)
            self._comm = None

    def abort(self) -> None:  # the reference's Drop aborts the communicator (src/eccl.rs:63-70)
        if self._comm:
            lib().ecclCommAbort(self._comm)
            self._comm = None


class OneShotAllReduce:
    """In-place bf16 sum over the ranks for small vectors, pushed over peer memory in one kernel
    (``ub_allreduce_oneshot_bf16``): the exchange after a row-split decode matmul, where the reference calls
    ``all_reduce`` (src/eccl.rs:209-245) and a library all-reduce is latency bound.

    ``exchange(obj)`` must return the list of every rank's ``obj`` in rank order (an all-gather over any
    out-of-band channel: a CPU process group, a shared list between threads).  With ``same_process`` the
    ranks are threads of one process: the peers' pointers are used directly after enabling peer access;
    otherwise the staging buffers are opened through IPC handles.  After construction every rank must pass
    a barrier of the caller's before the first ``all_reduce`` (all staging buffers zeroed and mapped)."""

    def __init__(self, dev, rank: int, world: int, max_bytes: int, exchange, same_process: bool = False):
        self.dev, self.rank, self.world, self.max_bytes = dev, rank, world, (max_bytes + 15) // 16 * 16
        nbytes = lib().ub_allreduce_oneshot_staging_bytes(world, self.max_bytes)
        if nbytes == 0:
            raise EcclError(4, "ub_allreduce_oneshot_staging_bytes")
        ptr = ctypes.c_void_p()
        _lib.check(lib().ub_p2p_alloc(nbytes, ctypes.byref(ptr)), "ub_p2p_alloc")  # on the thread's current device
        self._staging_ptr = ptr.value
        self._opened = []
        if same_process:
            infos = exchange((dev.ordinal, self._staging_ptr))
            ptrs = []
            for r, (ordinal, ptr) in enumerate(infos):
                if r != rank:
                    _lib.check(lib().ub_enable_peer_access(ordinal), "ub_enable_peer_access")
                ptrs.append(ptr)
        else:
            handle = ctypes.create_string_buffer(64)
            _lib.check(lib().ub_ipc_get_handle(ctypes.c_void_p(self._staging_ptr), handle), "ub_ipc_get_handle")
            handles = exchange(handle.raw)
            ptrs = []
            for r, raw in enumerate(handles):
                if r == rank:
                    ptrs.append(self._staging_ptr)
                    continue
                out = ctypes.c_void_p()
                _lib.check(lib().ub_ipc_open_handle(ctypes.create_string_buffer(raw, 64), ctypes.byref(out)),
                           "ub_ipc_open_handle")
                self._opened.append(out.value)
                ptrs.append(out.value)
        self._table = (ctypes.c_void_p * world)(*ptrs)

    def all_reduce(self, buf, count: int, stream=None) -> None:
        _lib.check(lib().ub_allreduce_oneshot_bf16(_p(buf), count, self._table, self.rank, self.world, self.max_bytes,
                                                   _p(stream if stream is not None else self.dev.stream)),
                   "ub_allreduce_oneshot_bf16")

    def matmul_all_reduce(self, y, x, wq, M: int, N: int, K: int, stream=None, residual=None) -> None:
        """y[M, N] (bf16) = [residual +] sum over the ranks of x_r[M, K] . W_r^T for a row-split Q4_K matrix,
        through ``ub_qmatmul_q4k_allreduce_residual_bf16``: with one token the exchange (and the residual add) is
        the matmul kernel's own epilogue."""
        _lib.check(lib().ub_qmatmul_q4k_allreduce_residual_bf16(
            _p(y), _p(x), _p(wq), _p(residual), M, N, K, self._table, self.rank, self.world, self.max_bytes,
            _p(stream if stream is not None else self.dev.stream)), "ub_qmatmul_q4k_allreduce_residual_bf16")

    def close(self) -> None:
        """Call after a barrier: no peer may still be pushing into this rank's buffer."""
        for p in self._opened:
            lib().ub_ipc_close_handle(ctypes.c_void_p(p))
        self._opened = []
        if self._staging_ptr:
            lib().ub_p2p_free(ctypes.c_void_p(self._staging_ptr))
            self._staging_ptr = None
