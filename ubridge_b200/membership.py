"""Host-side failure detection for ranks that run the sharded path.

A collective (or the peer-memory exchange inside a matmul) whose peer has gone away can only time out; the
ranks should learn of a departure on the HOST, before their next launch.  The reference leaves this to its
caller (one rank per process or thread, src/eccl.rs:155-206; a communicator is aborted when dropped,
src/eccl.rs:63-70).  ``StepGuard`` is the small protocol a caller needs, on top of any key-value store that
offers ``add(key, n) -> int`` and ``set(key, bytes)`` / ``get(key)`` (torch.distributed's TCPStore, FileStore
and HashStore do):

* ``join(timeout_s)``: every rank posts the world size it was started with; a rank that sees more joins than
  ranks of its own world size raises ``WorldMismatch`` at once, a rank whose world never fills raises
  ``RendezvousTimeout``;
* ``beat(step)`` after every step, ``check()`` before every launch: raises ``RankLeft`` when a rank has
  announced its departure with ``leave()`` (always between steps, with nothing in flight) and
  ``RankStale`` when a rank's last heartbeat is older than ``stale_after_s`` (a rank that died without a word).

Nothing here touches a GPU.
"""
from __future__ import annotations

import time


class MembershipError(RuntimeError):
    pass


class WorldMismatch(MembershipError):
    pass


class RendezvousTimeout(MembershipError):
    pass


class RankLeft(MembershipError):
    def __init__(self, ranks):
        super().__init__("ranks %s have left" % (sorted(ranks),))
        self.ranks = sorted(ranks)


class RankStale(MembershipError):
    def __init__(self, ranks):
        super().__init__("no heartbeat from ranks %s" % (sorted(ranks),))
        self.ranks = sorted(ranks)


class StepGuard:
    def __init__(self, store, rank: int, world: int, prefix: str = "ub", stale_after_s: float | None = None,
                 clock=time.time, sleep=time.sleep):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self.stale_after_s = stale_after_s
        self._clock, self._sleep = clock, sleep
        self._left_seen = 0

    def _k(self, *parts) -> str:
        return "/".join((self.prefix,) + tuple(str(p) for p in parts))

    # ---- rendezvous
    def join(self, timeout_s: float = 30.0, poll_s: float = 0.01) -> None:
        self.store.add(self._k("world", self.world), 1)
        self.store.add(self._k("joined"), 1)
        self.beat(-1)
        deadline = self._clock() + timeout_s
        while True:
            joined = self.store.add(self._k("joined"), 0)
            mine = self.store.add(self._k("world", self.world), 0)
            if joined > mine:
                raise WorldMismatch("rank %d was started with world size %d, but %d of the %d ranks that joined "
                                    "were started with another" % (self.rank, self.world, joined - mine, joined))
            if mine >= self.world:
                return
            if self._clock() >= deadline:
                raise RendezvousTimeout("rank %d: %d of %d ranks joined within %.1f s" %
                                        (self.rank, mine, self.world, timeout_s))
            self._sleep(poll_s)

    # ---- per step
    def beat(self, step: int) -> None:
        self.store.set(self._k("hb", self.rank), ("%d %.6f" % (step, self._clock())).encode())

    def leave(self) -> None:
        """Announce that this rank stops after the step it has completed.  Call with no kernel or collective of this
        rank in flight."""
        self.store.set(self._k("left", self.rank), b"1")
        self.store.add(self._k("left_count"), 1)

    def check(self) -> None:
        """Call before every launch that involves the other ranks."""
        n = self.store.add(self._k("left_count"), 0)
        if n > 0:
            raise RankLeft([r for r in range(self.world) if r != self.rank and self._has(self._k("left", r))])
        if self.stale_after_s is not None:
            now, stale = self._clock(), []
            for r in range(self.world):
                if r == self.rank:
                    continue
                key = self._k("hb", r)
                if not self._has(key):
                    stale.append(r)
                    continue
                t = float(bytes(self.store.get(key)).split()[1])
                if now - t > self.stale_after_s:
                    stale.append(r)
            if stale:
                raise RankStale(stale)

    def _has(self, key: str) -> bool:
        chk = getattr(self.store, "check", None)
        if chk is not None:
            return bool(chk([key]))
        try:
            self.store.get(key)
            return True
        except Exception:
            return False
