"""Rendezvous over a ``torch.distributed`` key-value store.

Plays the part of the reference's bridge records: node table, HELLO/LINK exchanges and the
membership *view* id that every plan carries (rdma/mesh-records.c:678-770; wire verbs
HELLO/LINK/ARRIVE in rdma/mesh-bridge.h:237-239).  On one NVSwitch node no sequencer is needed —
stream order and the per-communicator sequence number order everything — so what remains is:
exchange of small byte strings, host barriers with a "no progress" bound, an epoch word, and
passing file descriptors (VMM handles) between ranks over Unix sockets.
"""
from __future__ import annotations

import os
import pickle
import socket
import struct
import tempfile
import threading
import time
from typing import Any

ETIMEDOUT, ECANCELED, ESTALE = 110, 125, 116


class MeshHostTimeout(TimeoutError):
    errno = ETIMEDOUT


class MeshStale(RuntimeError):
    errno = ESTALE


class Rendezvous:
    """Rank table + byte exchange + barriers over a c10d Store (TCPStore, FileStore, HashStore)."""

    def __init__(self, store, rank: int, world: int, prefix: str = "mesh", timeout_s: float = 60.0):
        self.store = store
        self.rank = rank
        self.world = world
        self.prefix = prefix
        self.timeout_s = timeout_s
        self._seq = 0
        self.epoch = 0

    # ---- keys
    def _key(self, *parts) -> str:
        return "/".join([self.prefix, *map(str, parts)])

    def _wait_get(self, key: str) -> bytes:
        """Bounded get: polls so that a peer that never arrives raises instead of hanging."""
        deadline = time.monotonic() + self.timeout_s
        while True:
            try:
                if self.store.check([key]):
                    return self.store.get(key)
            except Exception:
                pass
            if time.monotonic() > deadline:
                raise MeshHostTimeout(f"rendezvous: key {key!r} not published within {self.timeout_s}s")
            time.sleep(0.002)

    def exchange(self, tag: str, payload: Any) -> list:
        """All-gather of one picklable object per rank."""
        self._seq += 1
        base = self._key("x", tag, self._seq)
        self.store.set(f"{base}/{self.rank}", pickle.dumps(payload))
        return [pickle.loads(self._wait_get(f"{base}/{r}")) for r in range(self.world)]

    def barrier(self, tag: str = "b") -> None:
        self.exchange("barrier-" + tag, self.rank)

    # ---- membership view
    def advance_epoch(self) -> int:
        """Agree on a new view id (max over ranks + 1).  Plans built under an older epoch are stale."""
        seen = self.exchange("epoch", self.epoch)
        self.epoch = max(seen) + 1
        return self.epoch

    def check_epoch(self, plan_epoch: int) -> None:
        if plan_epoch != self.epoch:
            raise MeshStale(f"plan was built for view {plan_epoch}, current view is {self.epoch}")

    # ---- file descriptors
    def exchange_fds(self, tag: str, fd: int) -> list[int]:
        """Every rank contributes one fd; returns the world's fds (own entry = the fd passed in).

        Descriptors travel as SCM_RIGHTS ancillary data over Unix stream sockets.
        """
        if self.world == 1:
            return [fd]
        path = os.path.join(tempfile.gettempdir(), f"mesh-{os.getpid()}-{self.rank}-{tag}-{self._seq}.sock")
        try:
            os.unlink(path)
        except FileNotFoundError:
            pass
        srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        srv.bind(path)
        srv.listen(self.world)
        srv.settimeout(self.timeout_s)
        got: dict[int, int] = {self.rank: fd}
        err: list[BaseException] = []

        def serve():
            try:
                for _ in range(self.world - 1):
                    conn, _ = srv.accept()
                    with conn:
                        conn.settimeout(self.timeout_s)
                        msg, fds, _, _ = socket.recv_fds(conn, 4, 1)
                        (src,) = struct.unpack("<i", msg)
                        got[src] = fds[0]
                        conn.sendall(b"k")
            except BaseException as e:  # reported to the caller below
                err.append(e)

        th = threading.Thread(target=serve, daemon=True)
        th.start()
        paths = self.exchange("fdpath-" + tag, path)
        for r in range(self.world):
            if r == self.rank:
                continue
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            c.settimeout(self.timeout_s)
            c.connect(paths[r])
            socket.send_fds(c, [struct.pack("<i", self.rank)], [fd])
            c.recv(1)
            c.close()
        th.join(self.timeout_s)
        srv.close()
        try:
            os.unlink(path)
        except FileNotFoundError:
            pass
        if err:
            raise err[0]
        if len(got) != self.world:
            raise MeshHostTimeout(f"fd exchange {tag}: got {len(got)} of {self.world}")
        return [got[r] for r in range(self.world)]


def from_process_group(group=None, prefix: str = "mesh") -> Rendezvous:
    """Build a Rendezvous from an initialised ``torch.distributed`` process group's store."""
    import torch.distributed as dist
    from torch.distributed import distributed_c10d as c10d
    if group is None:
        group = dist.group.WORLD
    store = c10d._get_default_store()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    uid = getattr(group, "group_name", "") or "world"
    from torch.distributed import PrefixStore
    return Rendezvous(PrefixStore(f"{prefix}/{uid}", store), rank, world, prefix="r")
