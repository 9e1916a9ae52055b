"""Python side of the per-process runtime service (csrc/runtime/runtime.cpp): start/stop, counters,
channel states, deadline, and reading any rank's stats block (what ``meshctl status`` prints)."""
from __future__ import annotations

import time
from ctypes import c_char_p, c_double, c_int, c_uint64

from .. import _native

CHANNEL = {0: "CLOSED", 1: "OPEN", 2: "MAPPED", 3: "CONNECTED", 4: "HALTED"}


def start(group: str, rank: int, world: int, heartbeat_s: float = 1.0) -> bool:
    """Returns True when an existing block of the same (group, rank, world) was re-adopted."""
    rc = _native.lib().mesh_runtime_start(c_char_p(group.encode()), c_int(rank), c_int(world), c_double(heartbeat_s))
    if rc < 0:
        raise OSError("mesh_runtime_start: cannot create the stats block")
    return rc == 1


def stop(unlink: bool = False) -> None:
    _native.lib().mesh_runtime_stop(c_int(int(unlink)))


def count(what: str, n: int = 1, peer: int = -1) -> None:
    idx = {"launches": 0, "collectives": 1, "timeouts": 2, "bytes": 3, "step": 4, "epoch": 5}[what]
    _native.lib().mesh_runtime_count(c_int(idx), c_uint64(n), c_int(peer))


def channel(peer: int, state: str) -> None:
    _native.lib().mesh_runtime_channel(c_int(peer), c_int({v: k for k, v in CHANNEL.items()}[state]))


def deadline(seconds: float) -> None:
    _native.lib().mesh_runtime_deadline(c_double(seconds))


def aborted() -> bool:
    return bool(_native.lib().mesh_runtime_aborted())


def abort(v: bool = True) -> None:
    _native.lib().mesh_runtime_abort(c_int(int(v)))


def read(group: str, rank: int) -> dict | None:
    out = (c_uint64 * 32)()
    rc = _native.lib().mesh_runtime_read(c_char_p(group.encode()), c_int(rank), out)
    if rc != 0:
        return None
    now = out[11]
    hb = out[4]
    return {
        "rank": int(out[0]), "world": int(out[1]), "pid": int(out[2]), "start_ns": int(out[3]),
        "heartbeat_age_s": (now - hb) / 1e9 if hb else None, "alive": bool(hb) and (now - hb) < 5e9,
        "epoch": int(out[5]), "step": int(out[6]), "launches": int(out[7]), "collectives": int(out[8]),
        "timeouts": int(out[9]), "abort": int(out[10]),
        "bytes_to_peer": [int(out[16 + i]) for i in range(8)],
        "channels": [CHANNEL.get(int(out[24 + i]), "?") for i in range(8)],
    }
