"""CPU: failure detection on the host, no GPU involved and no GPU fault provoked.

* a rank that leaves between steps is seen by the others through the store BEFORE their next collective;
* a rank that dies without a word shows up as a stale heartbeat;
* a world-size mismatch at rendezvous fails fast, a world that never fills fails within its timeout;
* Comm.wait bounds a collective by a host deadline and aborts the communicator (against fakes of the stream
  query, the asynchronous error state and the abort call)."""
import socket
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ubridge_b200 import _lib, eccl, membership as mb


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _store(rank, world, port):
    return dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20),
                         wait_for_workers=False)


def _leaver(rank, world, port, q):
    """Three ranks step together; rank 2 leaves after step 1.  The others must stop BEFORE entering step 2's
    all-reduce (which could only time out) and report who left."""
    store = _store(rank, world, port)
    guard = mb.StepGuard(store, rank, world)
    guard.join(timeout_s=20)
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world,
                            timeout=timedelta(seconds=20))
    steps_done, seen = 0, None
    try:
        for step in range(4):
            if rank == 2 and step == 2:
                guard.leave()  # between steps, nothing in flight
                break
            # the step's own all-reduce doubles as the point after which a departure becomes visible
            if step == 2:
                deadline = time.time() + 10
                while time.time() < deadline:  # the leaver announces within moments of finishing step 1
                    try:
                        guard.check()
                    except mb.RankLeft as e:
                        seen = e.ranks
                        break
                    time.sleep(0.01)
                if seen is not None:
                    break
            guard.check()
            t = torch.ones(4) * (rank + 1)
            dist.all_reduce(t)
            assert float(t[0]) == 6.0
            guard.beat(step)
            steps_done += 1
    finally:
        q.put((rank, steps_done, seen))
        # the survivors do not call into the process group again; rank 0 keeps the store alive until all reported
        if rank == 0:
            deadline = time.time() + 10
            while store.add("reported", 0) < world - 1 and time.time() < deadline:
                time.sleep(0.01)
        else:
            store.add("reported", 1)


def test_rank_leaving_between_steps_is_seen_before_the_next_launch():
    world, port = 3, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_leaver, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    assert out[0] == (0, 2, [2]) and out[1] == (1, 2, [2])
    assert out[2] == (2, 2, None)


class DictStore:
    """In-process store with the three calls StepGuard uses."""

    def __init__(self):
        self.kv, self.cnt = {}, {}

    def add(self, key, n):
        self.cnt[key] = self.cnt.get(key, 0) + n
        return self.cnt[key]

    def set(self, key, val):
        self.kv[key] = bytes(val)

    def get(self, key):
        return self.kv[key]

    def check(self, keys):
        return all(k in self.kv for k in keys)


class FakeTime:
    def __init__(self):
        self.t = 1000.0

    def clock(self):
        return self.t

    def sleep(self, s):
        self.t += s


def test_world_size_mismatch_fails_fast_and_short_world_times_out():
    store, ft = DictStore(), FakeTime()
    a = mb.StepGuard(store, 0, 2, clock=ft.clock, sleep=ft.sleep)
    b = mb.StepGuard(store, 1, 3, clock=ft.clock, sleep=ft.sleep)  # started with the wrong world size
    with pytest.raises(mb.RendezvousTimeout):
        a.join(timeout_s=0.5)  # alone: the world never fills
    with pytest.raises(mb.WorldMismatch):
        b.join(timeout_s=5.0)  # sees a join that is not of its world size
    with pytest.raises(mb.WorldMismatch):
        mb.StepGuard(store, 0, 2, clock=ft.clock, sleep=ft.sleep).join(timeout_s=5.0)


def test_stale_heartbeat_marks_a_rank_that_died_silently():
    store, ft = DictStore(), FakeTime()
    g0 = mb.StepGuard(store, 0, 2, stale_after_s=1.0, clock=ft.clock, sleep=ft.sleep)
    g1 = mb.StepGuard(store, 1, 2, stale_after_s=1.0, clock=ft.clock, sleep=ft.sleep)
    store.add("ub/world/2", 1), store.add("ub/joined", 1)  # rank 1 has joined already
    g1.beat(-1)
    g0.join(timeout_s=1.0)
    g0.check()
    ft.sleep(0.6)
    g1.beat(0)
    ft.sleep(0.6)
    g0.check()  # 0.6 s since rank 1's last beat
    ft.sleep(0.6)
    with pytest.raises(mb.RankStale) as ei:
        g0.check()
    assert ei.value.ranks == [1]
    g1.leave()
    with pytest.raises(mb.RankLeft) as ei:
        g0.check()
    assert ei.value.ranks == [1]


class FakeComm(eccl.Comm):
    def __init__(self, errors):
        super().__init__(handle=None, rank=0, world_size=2)
        self.errors, self.aborted = list(errors), 0

    def async_error(self):
        return self.errors.pop(0) if self.errors else 0

    def abort(self):
        self.aborted += 1


def test_wait_returns_when_the_stream_drains():
    ft, c = FakeTime(), FakeComm([])
    answers = [_lib.UB_ERR_NOT_READY] * 3 + [_lib.UB_OK]
    c.wait(None, 1.0, query=lambda: answers.pop(0), clock=ft.clock, sleep=ft.sleep)
    assert c.aborted == 0 and not answers


def test_wait_aborts_on_deadline():
    ft, c = FakeTime(), FakeComm([])
    with pytest.raises(eccl.EcclTimeout):
        c.wait(None, 0.05, poll_s=0.01, query=lambda: _lib.UB_ERR_NOT_READY, clock=ft.clock, sleep=ft.sleep)
    assert c.aborted == 1
    assert ft.t - 1000.0 < 0.1  # gave up at the deadline, not later


def test_wait_aborts_on_asynchronous_error_and_on_stream_error():
    ft, c = FakeTime(), FakeComm([0, 7, 6])  # success, in progress, remote error
    with pytest.raises(eccl.EcclError) as ei:
        c.wait(None, 10.0, query=lambda: _lib.UB_ERR_NOT_READY, clock=ft.clock, sleep=ft.sleep)
    assert ei.value.code == 6 and c.aborted == 1 and not isinstance(ei.value, eccl.EcclTimeout)
    c2 = FakeComm([])
    with pytest.raises(eccl.EcclError) as ei:
        c2.wait(None, 10.0, query=lambda: _lib.UB_ERR_CUDA, clock=ft.clock, sleep=ft.sleep)
    assert ei.value.code == _lib.UB_ERR_CUDA and c2.aborted == 1
