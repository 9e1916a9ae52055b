"""``python -m mesh_b200.tools.meshctl status|top [--group G] [--world N]``

Reads every rank's stats block (shared memory written by the runtime service) without touching the
GPUs: liveness, epoch, step, launches, collectives, timeouts, bytes per peer and channel states — the
reference's ``mesh-stat`` (rdma/mesh-stat.c:65-118) and ``mesh-top`` (bin/mesh-top.py) for one NVSwitch node.
``--ready`` exits 0 only when every rank is alive and none has its abort flag up.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def snapshot(group: str, world: int) -> list:
    from ..runtime import service
    return [service.read(group, r) for r in range(world)]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="meshctl")
    ap.add_argument("command", choices=["status", "top"])
    ap.add_argument("--group", default="mesh")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--ready", action="store_true")
    ap.add_argument("--interval", type=float, default=1.0)
    ap.add_argument("--count", type=int, default=0, help="top: number of refreshes (0 = until interrupted)")
    a = ap.parse_args(argv)
    if a.command == "status":
        snap = snapshot(a.group, a.world)
        print(json.dumps({"group": a.group, "ranks": snap}, indent=1))
        if a.ready:
            ok = all(s is not None and s["alive"] and not s["abort"] for s in snap)
            return 0 if ok else 1
        return 0
    prev, n = None, 0
    while True:
        snap = snapshot(a.group, a.world)
        lines = [f"{'rank':>4} {'alive':>5} {'epoch':>5} {'step':>8} {'launch/s':>9} {'coll/s':>8} {'timeouts':>8} {'MB/s out':>9}"]
        for r, s in enumerate(snap):
            if s is None:
                lines.append(f"{r:>4} {'-':>5}")
                continue
            p = prev[r] if prev and prev[r] else None
            rate = lambda k: (s[k] - p[k]) / a.interval if p else 0.0
            mb = (sum(s["bytes_to_peer"]) - sum(p["bytes_to_peer"])) / a.interval / 1e6 if p else 0.0
            lines.append(f"{r:>4} {str(s['alive']):>5} {s['epoch']:>5} {s['step']:>8} {rate('launches'):>9.0f} "
                         f"{rate('collectives'):>8.0f} {s['timeouts']:>8} {mb:>9.1f}")
        sys.stdout.write("\n".join(lines) + "\n")
        sys.stdout.flush()
        prev = snap
        n += 1
        if a.count and n >= a.count:
            return 0
        time.sleep(a.interval)


if __name__ == "__main__":
    sys.exit(main())
