"""Peer channels (``csrc/runtime/peer_channel.cu``): per-peer state, copy-engine transfers served by a proxy thread,
bounded flush.  See the C++ file for what a channel is for on NVLink."""
from __future__ import annotations

from ctypes import c_int, c_uint64, c_void_p

from .. import _native

STATES = {0: "CLOSED", 1: "OPEN", 2: "MAPPED", 3: "CONNECTED", 4: "HALTED"}
_CODE = {v: k for k, v in STATES.items()}


class ChannelError(RuntimeError):
    pass


class PeerChannels:
    """``device``: CUDA device index, or ``-1`` for host-memory channels (tests without a GPU)."""

    def __init__(self, rank: int, world: int, device: int = -1):
        L = _native.lib()
        L.mesh_channels_create.restype = c_void_p
        L.mesh_channel_copy.restype = c_uint64
        L.mesh_channel_bytes.restype = c_uint64
        self.L, self.rank, self.world = L, rank, world
        self.h = c_void_p(L.mesh_channels_create(c_int(rank), c_int(world), c_int(device)))
        if not self.h:
            raise ChannelError(_native.last_error())

    def advance(self, peer: int, state: str) -> None:
        if self.L.mesh_channel_advance(self.h, c_int(peer), c_int(_CODE[state])) != 0:
            raise ChannelError(_native.last_error())

    def connect_all(self) -> None:
        """Every peer's memory is mapped (the symmetric heap exists): OPEN -> MAPPED -> CONNECTED."""
        for p in range(self.world):
            if self.state(p) == "OPEN":
                self.advance(p, "MAPPED")
            if self.state(p) == "MAPPED":
                self.advance(p, "CONNECTED")

    def state(self, peer: int) -> str:
        return STATES.get(self.L.mesh_channel_state(self.h, c_int(peer)), "?")

    def copy(self, peer: int, dst: int, src: int, nbytes: int, after_stream: int = 0) -> int:
        """Queue ``nbytes`` from address ``src`` to ``dst`` on the channel to ``peer``; returns the job's ticket."""
        t = int(self.L.mesh_channel_copy(self.h, c_int(peer), c_void_p(dst), c_void_p(src), c_uint64(nbytes), c_void_p(after_stream)))
        if t == 0:
            raise ChannelError(_native.last_error())
        return t

    def done(self, peer: int, ticket: int) -> bool:
        r = self.L.mesh_channel_done(self.h, c_int(peer), c_uint64(ticket))
        if r < 0:
            raise ChannelError(f"channel {peer} halted before job {ticket} finished")
        return r == 1

    def wait_on_stream(self, peer: int, ticket: int, stream: int, timeout_ms: int = 5000) -> None:
        if self.L.mesh_channel_wait_on_stream(self.h, c_int(peer), c_uint64(ticket), c_void_p(stream), c_int(timeout_ms)) != 0:
            raise ChannelError(_native.last_error())

    def flush(self, timeout_ms: int = 5000) -> int:
        """Waits (bounded) for channels with outstanding work; returns how many it had to halt."""
        return int(self.L.mesh_channels_flush(self.h, c_int(timeout_ms)))

    def bytes(self, peer: int) -> int:
        return int(self.L.mesh_channel_bytes(self.h, c_int(peer)))

    def close(self, timeout_ms: int = 5000) -> int:
        if not self.h:
            return 0
        n = int(self.L.mesh_channels_destroy(self.h, c_int(timeout_ms)))
        self.h = None
        return n

    def __del__(self):
        try:
            self.close(1000)
        except Exception:
            pass
