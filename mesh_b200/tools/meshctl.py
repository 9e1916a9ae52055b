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
        sys.stdout.write(render_top(a.group, snap, prev, a.interval) + "\n")
        sys.stdout.flush()
        prev = snap
        n += 1
        if a.count and n >= a.count:
            return 0
        time.sleep(a.interval)


def render_top(group: str, snap: list, prev: list | None, interval: float) -> str:
    """One screen of ``meshctl top``: a line per rank (liveness, heartbeat age, view, step, launches / collectives per
    second, timeouts, abort flag), then the matrix of bytes per second that each rank's links carry to each peer and
    the state of every peer channel - the nodes / rates / links / communicators panes of the reference's ``mesh-top``
    (bin/mesh-top.py) for one NVSwitch node."""
    world = len(snap)
    lines = [f"group {group}   ranks {sum(1 for s in snap if s and s['alive'])}/{world} alive   "
             f"aborted {sum(1 for s in snap if s and s['abort'])}",
             f"{'rank':>4} {'alive':>5} {'hb age':>7} {'view':>5} {'step':>8} {'launch/s':>9} {'coll/s':>8} {'timeouts':>8} {'abort':>5} {'MB/s out':>9}"]
    rates = []
    for r, s in enumerate(snap):
        if s is None:
            lines.append(f"{r:>4} {'-':>5}   (no stats block)")
            rates.append(None)
            continue
        p = prev[r] if prev and r < len(prev) and prev[r] else None
        rate = (lambda k: (s[k] - p[k]) / interval) if p else (lambda k: 0.0)
        per_peer = [((s["bytes_to_peer"][i] - p["bytes_to_peer"][i]) / interval / 1e6 if p else 0.0) for i in range(min(world, 8))]
        rates.append(per_peer)
        age = s["heartbeat_age_s"]
        lines.append(f"{r:>4} {str(s['alive']):>5} {('%.1fs' % age) if age is not None else '-':>7} {s['epoch']:>5} {s['step']:>8} "
                     f"{rate('launches'):>9.0f} {rate('collectives'):>8.0f} {s['timeouts']:>8} {s['abort']:>5} {sum(per_peer):>9.1f}")
    lines.append("links (MB/s, row = sender, column = peer):")
    lines.append("      " + " ".join(f"{c:>8}" for c in range(min(world, 8))))
    for r, row in enumerate(rates):
        lines.append(f"{r:>4}  " + (" ".join(f"{v:>8.1f}" for v in row) if row is not None else "-"))
    lines.append("channels (row = rank, column = peer): " + "  ".join(
        f"{r}:[" + ",".join(c[:4] for c in s["channels"][:min(world, 8)]) + "]" for r, s in enumerate(snap) if s is not None))
    return "\n".join(lines)


if __name__ == "__main__":
    sys.exit(main())
