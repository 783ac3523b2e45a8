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
