"""GPU: the ECCL-shaped collectives over NCCL.  Threads stand for ranks, one per device, the pattern of
the reference's own collective tests (src/eccl.rs:428-492: all-reduce of [(i+1); 2] expects n(n+1)/2)."""
import threading

import numpy as np
import pytest

import ubridge_b200 as ub
from ubridge_b200 import eccl

pytestmark = pytest.mark.gpu


def test_version_and_unique_id():
    assert eccl.get_version() >= 20000
    a, b = eccl.Id(), eccl.Id()
    assert len(a.internal()) == 128 and a.internal() != b.internal()
    assert eccl.Id.uninit(a.internal()).internal() == a.internal()


def test_single_rank_collectives(dev):
    dev.bind_to_thread()
    comm = eccl.Comm.from_rank(0, 1, eccl.Id())
    assert comm.count() == 1 and comm.user_rank() == 0 and comm.device() == dev.ordinal
    x = np.arange(1000, dtype=np.float32)
    d_x, d_y = dev.htod_sync_copy(x), dev.alloc(x.nbytes)
    comm.all_reduce(d_x, d_y, x.size, eccl.Float32, eccl.ReduceOp.Sum, stream=dev.stream)
    assert np.array_equal(dev.dtoh_sync_copy(d_y, np.float32), x)
    comm.all_gather(d_x, d_y, x.size, eccl.Float32, stream=dev.stream)
    assert np.array_equal(dev.dtoh_sync_copy(d_y, np.float32), x)
    comm.broadcast(d_x, d_y, x.size, eccl.Float32, 0, stream=dev.stream)
    # the host's deadline-bounded wait: polls the stream and the communicator's asynchronous error state
    comm.wait(dev.stream, 10.0)
    assert comm.async_error() == 0
    assert ub.lib().ub_stream_query(dev.stream) == 0  # drained
    dev.synchronize()
    comm.destroy()


def test_all_reduce_across_devices_threads_as_ranks():
    n = ub.lib().ub_device_count()
    if n < 2:
        pytest.skip("needs 2+ GPUs")
    n = min(n, 4)
    uid = eccl.Id()
    results = [None] * n

    def rank_main(r):
        d = ub.GcuDevice(r)
        d.bind_to_thread()
        comm = eccl.Comm.from_rank(r, n, uid)
        x = np.full(2, r + 1, dtype=np.float32)
        d_x, d_y = d.htod_sync_copy(x), d.alloc(8)
        comm.all_reduce(d_x, d_y, 2, eccl.Float32, eccl.ReduceOp.Sum, stream=d.stream)
        results[r] = d.dtoh_sync_copy(d_y, np.float32)
        comm.destroy()

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    for r in range(n):
        assert results[r] is not None and (results[r] == n * (n + 1) / 2).all()


def test_one_shot_all_reduce_gives_up_when_a_rank_never_arrives(dev):
    """Failure detection without a fault: world = 2 with both staging buffers on this GPU, only rank 0 ever
    launches, so rank 1's flag is never raised.  With a small poll limit the wait runs out in well under a
    second, the kernel returns, the context stays usable and the device error word reads UB_ERR_TIMEOUT."""
    import ctypes
    import time

    from ubridge_b200._lib import UB_ERR_TIMEOUT, check, lib

    dev.bind_to_thread()
    dev.synchronize()
    assert dev.device_status() == 0
    world, max_bytes, count = 2, 4096, 1024
    nbytes = lib().ub_allreduce_oneshot_staging_bytes(world, max_bytes)
    bufs = []
    for _ in range(world):
        p = ctypes.c_void_p()
        check(lib().ub_p2p_alloc(nbytes, ctypes.byref(p)), "ub_p2p_alloc")
        bufs.append(p.value)
    table = (ctypes.c_void_p * world)(*bufs)
    x = np.ones(count, dtype=np.uint16) * 0x3F80  # bf16 1.0
    d_x = dev.htod_sync_copy(x)
    prev = lib().ub_allreduce_oneshot_set_spin_limit(2000)
    try:
        t0 = time.perf_counter()
        check(lib().ub_allreduce_oneshot_bf16(ctypes.c_void_p(d_x.ptr), count, table, 0, world, max_bytes, dev.stream),
              "ub_allreduce_oneshot_bf16")
        dev.synchronize()
        assert time.perf_counter() - t0 < 1.0
        assert dev.device_status() == UB_ERR_TIMEOUT  # read and clear
        assert dev.device_status() == 0
        # the context is intact: an ordinary copy still works
        assert np.array_equal(dev.dtoh_sync_copy(dev.htod_sync_copy(x), np.uint16), x)
    finally:
        lib().ub_allreduce_oneshot_set_spin_limit(prev)
        for p in bufs:
            lib().ub_p2p_free(ctypes.c_void_p(p))
