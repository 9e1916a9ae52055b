"""Failure detection and elastic regrouping — host side only.

The reference's "one failure detector" is holder identity (pid, start time) plus bounded waits everywhere
(rdma/mesh-holders.h:17-37; ETIMEDOUT / ESTALE / ECANCELED, rdma/mesh.h:15-17), membership *views* that make old
plans stale (rdma/mesh-records.c:678-770), and a supervisor that restarts after an unasked exit
(rdma/mesh-heartbeat.c:5-30).  Here: every rank writes a heartbeat into the rendezvous store before each step
and reads its peers'; a rank that leaves announces it (or simply stops beating); survivors learn of it on the
host before their next launch, raise ``PeerLost`` instead of entering a collective, agree on the surviving set,
bump the epoch (old plans become stale) and continue at the smaller world from the last checkpoint.
No GPU is faulted, trapped or hung to exercise any of this: failures are injected on the host.
"""
from __future__ import annotations

import os
import pickle
import time


class PeerLost(RuntimeError):
    def __init__(self, lost: list[int]):
        self.lost = lost
        super().__init__(f"ranks {lost} left the job")


def process_identity(pid: int | None = None) -> tuple[int, int]:
    """(pid, start time in clock ticks): survives pid reuse, like the reference's holder identity."""
    pid = pid or os.getpid()
    try:
        with open(f"/proc/{pid}/stat") as f:
            fields = f.read().rsplit(")", 1)[1].split()
        return pid, int(fields[19])
    except Exception:
        return pid, 0


def alive(identity: tuple[int, int]) -> bool:
    pid, start = identity
    cur = process_identity(pid)
    return cur[1] == start and start != 0 and os.path.exists(f"/proc/{pid}")


class FailureDetector:
    """Heartbeats + departures over a c10d store."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "fd"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix
        self.members = list(range(world))
        self.epoch = 0
        self.beat()

    def _k(self, *parts) -> str:
        return "/".join([self.prefix, str(self.epoch), *map(str, parts)])

    def beat(self, step: int = 0) -> None:
        self.store.set(self._k("hb", self.rank), pickle.dumps((time.time(), step, process_identity())))

    def leave(self) -> None:
        """Announce an orderly departure (called between steps, with nothing in flight)."""
        self.store.set(self._k("left", self.rank), b"1")

    def check(self, step: int = 0) -> None:
        """Call before every step: beats, then raises ``PeerLost`` if a member announced leaving or went silent."""
        self.beat(step)
        lost = []
        now = time.time()
        for r in self.members:
            if r == self.rank:
                continue
            if self.store.check([self._k("left", r)]):
                lost.append(r)
                continue
            if self.store.check([self._k("hb", r)]):
                t, _, _ = pickle.loads(self.store.get(self._k("hb", r)))
                if now - t > self.timeout_s:
                    lost.append(r)
            elif now - getattr(self, "_t0", now) > self.timeout_s:
                lost.append(r)
        if not hasattr(self, "_t0"):
            self._t0 = now
        if lost:
            raise PeerLost(lost)

    def regroup(self, lost: list[int]) -> tuple[int, int, list[int]]:
        """Survivors agree on the new membership: returns ``(new rank, new world, members)`` and advances the epoch."""
        survivors = [r for r in self.members if r not in lost]
        old_epoch = self.epoch
        key = "/".join([self.prefix, str(old_epoch), "regroup", ",".join(map(str, survivors))])
        self.store.add(key, 1)
        deadline = time.time() + self.timeout_s * 4
        while int(self.store.add(key, 0)) < len(survivors):
            if time.time() > deadline:
                raise TimeoutError("regroup: not every survivor arrived")
            time.sleep(0.005)
        self.members = survivors
        self.epoch = old_epoch + 1
        self._t0 = time.time()
        self.beat()
        return survivors.index(self.rank), len(survivors), survivors
