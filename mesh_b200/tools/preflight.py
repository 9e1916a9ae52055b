"""Pre-run probe: ``python -m mesh_b200.tools.preflight --world 8 [--group G] [--port 29500]``.

Answers, before a job starts and without launching a kernel: which GPUs are visible and how much memory is free on
each, which other processes hold them, whether every pair of GPUs can map each other's memory, whether stats blocks of
an earlier job with the same group name are still attached to live processes (a collision) or are leftovers of dead
ones (removed with ``--clean``), whether the rendezvous port is free, and whether the native library is built for this
source tree.  Exit code 0: clear to run; 1: a collision or a missing resource, listed under ``problems``.
Counterpart of the reference's preflight (rdma/mesh_preflight.py:64-170: who holds the region and devices, beacons,
cables, collision detection).
"""
from __future__ import annotations

import argparse
import json
import os
import socket


def gpu_inventory(nvml=None) -> list[dict]:
    """One record per GPU: index, name, free / total MiB, compute processes.  ``nvml``: a ``pynvml``-like module."""
    out = []
    if nvml is None:
        try:
            import pynvml as nvml
            nvml.nvmlInit()
        except Exception:
            return out
    for i in range(nvml.nvmlDeviceGetCount()):
        h = nvml.nvmlDeviceGetHandleByIndex(i)
        mem = nvml.nvmlDeviceGetMemoryInfo(h)
        try:
            procs = [{"pid": p.pid, "mib": (p.usedGpuMemory or 0) >> 20} for p in nvml.nvmlDeviceGetComputeRunningProcesses(h)]
        except Exception:
            procs = []
        name = nvml.nvmlDeviceGetName(h)
        out.append({"gpu": i, "name": name.decode() if isinstance(name, bytes) else name, "free_mib": mem.free >> 20,
                    "total_mib": mem.total >> 20, "processes": procs})
    return out


def peer_matrix(n: int) -> list[list[bool]] | None:
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        n = min(n, torch.cuda.device_count())
        return [[a == b or bool(torch.cuda.can_device_access_peer(a, b)) for b in range(n)] for a in range(n)]
    except Exception:
        return None


def stats_blocks(group: str, world: int) -> list[dict]:
    """State of the named stats blocks of ``group``: absent, held by a live process, or left by a dead one."""
    from ..runtime import service
    out = []
    for r in range(world):
        s = service.read(group, r)
        if s is None:
            out.append({"rank": r, "state": "absent"})
        else:
            out.append({"rank": r, "state": "live" if s["alive"] else "stale", "pid": s.get("pid")})
    return out


def port_free(port: int, host: str = "127.0.0.1") -> bool:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((host, port))
            return True
        except OSError:
            return False


def probe(world: int, group: str = "mesh", port: int | None = None, min_free_mib: int = 8192, nvml=None,
          peers=None, blocks=None) -> dict:
    """The report.  ``nvml`` / ``peers`` / ``blocks`` can be injected (tests)."""
    gpus = gpu_inventory(nvml)
    rep = {"world": world, "group": group, "gpus": gpus, "problems": []}
    if gpus and len(gpus) < world:
        rep["problems"].append(f"{world} ranks wanted, {len(gpus)} GPUs visible")
    mine = os.getpid()
    for g in gpus[:world]:
        if g["free_mib"] < min_free_mib:
            rep["problems"].append(f"GPU {g['gpu']}: {g['free_mib']} MiB free, {min_free_mib} wanted")
        others = [p for p in g["processes"] if p["pid"] != mine]
        if others:
            rep["problems"].append(f"GPU {g['gpu']} is held by " + ", ".join(f"pid {p['pid']} ({p['mib']} MiB)" for p in others))
    pm = peers if peers is not None else peer_matrix(world)
    rep["peer_access"] = pm
    if pm is not None:
        bad = [(a, b) for a in range(len(pm)) for b in range(len(pm)) if not pm[a][b]]
        if bad:
            rep["problems"].append("no peer access between " + ", ".join(f"{a}-{b}" for a, b in bad[:8]))
    bl = blocks if blocks is not None else stats_blocks(group, world)
    rep["stats_blocks"] = bl
    live = [b for b in bl if b["state"] == "live"]
    if live:
        rep["problems"].append(f"group {group!r} is in use: ranks {[b['rank'] for b in live]} are attached to live processes")
    rep["stale_ranks"] = [b["rank"] for b in bl if b["state"] == "stale"]
    if port is not None:
        rep["port_free"] = port_free(port)
        if not rep["port_free"]:
            rep["problems"].append(f"port {port} is taken")
    try:
        from .. import _build
        rep["library_current"] = bool(_build.is_current()) if hasattr(_build, "is_current") else None
    except Exception:
        rep["library_current"] = None
    rep["ok"] = not rep["problems"]
    return rep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mesh-preflight")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--group", default="mesh")
    ap.add_argument("--port", type=int, default=None)
    ap.add_argument("--min-free-mib", type=int, default=8192)
    ap.add_argument("--clean", action="store_true", help="remove stats blocks left by dead processes")
    a = ap.parse_args(argv)
    rep = probe(a.world, a.group, a.port, a.min_free_mib)
    if a.clean and rep["stale_ranks"]:
        for r in rep["stale_ranks"]:
            try:
                os.unlink(f"/dev/shm/mesh_b200_{a.group}_{r}")
            except OSError:
                pass
        rep["cleaned"] = rep["stale_ranks"]
    print(json.dumps(rep, indent=1))
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
