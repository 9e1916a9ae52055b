"""Disk-room guard: every writer checks that the volume keeps a reserve before it writes
(rdma/mesh_disk.py:42, rdma/mesh-disk.h:28-60: refuse when the volume is nearly full)."""
from __future__ import annotations

import os
import shutil
from pathlib import Path

RESERVE_BYTES = 1 << 30
RESERVE_FRACTION = 0.02


class DiskFull(OSError):
    pass


def room(path, need: int = 0) -> int:
    """Free bytes available to writers at ``path`` after the reserve; raises ``DiskFull`` when ``need`` does not fit."""
    p = Path(path)
    while not p.exists() and p != p.parent:
        p = p.parent
    u = shutil.disk_usage(p)
    reserve = max(RESERVE_BYTES if u.total > 8 * RESERVE_BYTES else 0, int(u.total * RESERVE_FRACTION))
    free = u.free - reserve
    if need > free:
        raise DiskFull(f"{path}: need {need} bytes, {max(free, 0)} available after the reserve of {reserve}")
    return free
