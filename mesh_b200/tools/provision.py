"""Node convergence: ``python -m mesh_b200.tools.provision [--root DIR] [--apply] [--gpus N] [--keys FILE]``.

Brings a Linux GPU node to the state the package's services expect, idempotently: a second run changes nothing.  The
desired state is a list of items, each a file with exact content (systemd units for the telemetry provider and the
hourly health run with its timer, the environment file the units read, the fleet's authorised ssh keys, the runtime
identity record) plus read-only checks (interpreter, compiler, driver and GPU count seen through NVML).  Without
``--apply`` the tool only reports what differs (exit code 1 when something does); with it, it writes what differs under
``--root`` (default ``/``; a staging directory for images and tests) and nothing else.

It never changes a GPU's settings: clocks, power limits, persistence, MIG, compute and ECC modes are read and reported
only, since whoever gets the GPU next inherits them.  The reference converges its Macs the same idempotent way
(``install.sh``: launchd jobs, sshd, authorised keys, self-update; ``bin/mesh-runtime-install.sh``, ``bin/mesh-keeper.sh``);
the macOS-specific parts (launchctl, power policy, auto-login) have no counterpart on a Linux GPU node.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import sys
from dataclasses import dataclass
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]


@dataclass
class Item:
    path: str            # absolute path on the node (placed under --root)
    content: str
    mode: int = 0o644
    why: str = ""


def _unit(description: str, exec_start: str, env_file: str, extra: str = "") -> str:
    return (f"[Unit]\nDescription={description}\nAfter=network-online.target\n\n"
            f"[Service]\nType=simple\nEnvironmentFile=-{env_file}\nWorkingDirectory={REPO}\nExecStart={exec_start}\n"
            f"Restart=on-failure\nRestartSec=5\n{extra}\n[Install]\nWantedBy=multi-user.target\n")


def desired(gpus: int, keys: str | None, python: str = sys.executable, prefix: str = "/etc/mesh_b200") -> list[Item]:
    """The files of a converged node."""
    env = f"{prefix}/env"
    items = [
        Item(env, f"MESH_HOME={REPO}\nMESH_GPUS={gpus}\nMESH_RUNTIME=1\nPYTHONUNBUFFERED=1\n",
             why="environment of the services (MESH_* switches of docs/running.md go here)"),
        Item("/etc/systemd/system/mesh-telemetry.service",
             _unit("mesh_b200 telemetry provider (GPU, rank and workload state over HTTP)",
                   f"{python} -m mesh_b200.tools.telemetry --host 0.0.0.0 --port 8101", env),
             why="what `tools/observe.py` and `meshctl top` on other nodes read"),
        Item("/etc/systemd/system/mesh-hourly.service",
             ("[Unit]\nDescription=mesh_b200 scheduled health run\n\n[Service]\nType=oneshot\n"
              f"EnvironmentFile=-{env}\nWorkingDirectory={REPO}\n"
              f"ExecStart={python} -m mesh_b200.tools.hourly --gpus {gpus} --out /var/log/mesh_b200/hourly.jsonl\n"),
             why="regressions noticed by the node itself"),
        Item("/etc/systemd/system/mesh-hourly.timer",
             "[Unit]\nDescription=hourly mesh_b200 health run\n\n[Timer]\nOnCalendar=hourly\nPersistent=true\n\n"
             "[Install]\nWantedBy=timers.target\n", why="the timer of the health run"),
        Item(f"{prefix}/runtime.json", json.dumps(_runtime_identity(), indent=1, sort_keys=True) + "\n",
             why="which build of the package this node runs (compared across the fleet by `tools/fleet.py`)"),
    ]
    if keys:
        text = Path(keys).read_text()
        if not text.endswith("\n"):
            text += "\n"
        items.append(Item("/etc/ssh/authorized_keys.d/mesh_fleet", text, 0o600, "keys the fleet commands log in with"))
    return items


def _runtime_identity() -> dict:
    try:
        from .runtime_id import identity
        return identity()
    except Exception:
        h = hashlib.sha256()
        for p in sorted((REPO / "mesh_b200").rglob("*.py")):
            h.update(p.read_bytes())
        return {"sources": h.hexdigest()[:16]}


def checks(gpus: int, nvml=None) -> list[dict]:
    """Read-only facts about the node, each with ``ok``."""
    out = [{"check": "python >= 3.10", "ok": sys.version_info >= (3, 10), "seen": sys.version.split()[0]},
           {"check": "nvcc on PATH (the library is built in-tree)", "ok": bool(shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc")),
            "seen": shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"}]
    try:
        import torch
        out.append({"check": "torch importable", "ok": True, "seen": torch.__version__})
    except Exception as e:  # pragma: no cover - torch is a hard dependency everywhere else
        out.append({"check": "torch importable", "ok": False, "seen": str(e)})
    from .preflight import gpu_inventory
    gpus_seen = gpu_inventory(nvml)
    out.append({"check": f"{gpus} GPU(s) visible", "ok": len(gpus_seen) >= gpus, "seen": len(gpus_seen)})
    out.append({"check": "GPU settings (read only, never changed)", "ok": True, "seen": gpu_settings(nvml)})
    return out


def gpu_settings(nvml=None) -> list[dict]:
    """Persistence mode, power limit and SM clocks of every GPU as they are: reported, never set."""
    if nvml is None:
        try:
            import pynvml as nvml
            nvml.nvmlInit()
        except Exception:
            return []
    out = []
    for i in range(nvml.nvmlDeviceGetCount()):
        h = nvml.nvmlDeviceGetHandleByIndex(i)
        rec = {"gpu": i}
        for key, fn in (("persistence", "nvmlDeviceGetPersistenceMode"), ("power_limit_mw", "nvmlDeviceGetPowerManagementLimit")):
            try:
                rec[key] = getattr(nvml, fn)(h)
            except Exception:
                rec[key] = None
        out.append(rec)
    return out


def diff(items: list[Item], root: Path) -> list[dict]:
    """What separates the node (under ``root``) from the desired state."""
    out = []
    for it in items:
        p = root / it.path.lstrip("/")
        if not p.exists():
            out.append({"path": it.path, "change": "create", "why": it.why})
        elif p.read_text() != it.content:
            out.append({"path": it.path, "change": "rewrite", "why": it.why})
        elif (p.stat().st_mode & 0o777) != it.mode:
            out.append({"path": it.path, "change": "chmod", "why": it.why})
    return out


def apply(items: list[Item], root: Path) -> list[dict]:
    """Write what differs, file by file, each through a temporary name in the same directory."""
    changed = diff(items, root)
    wanted = {c["path"] for c in changed}
    for it in items:
        if it.path not in wanted:
            continue
        p = root / it.path.lstrip("/")
        p.parent.mkdir(parents=True, exist_ok=True)
        tmp = p.with_name(p.name + ".tmp")
        tmp.write_text(it.content)
        os.chmod(tmp, it.mode)
        os.replace(tmp, p)
    return changed


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mesh-provision")
    ap.add_argument("--root", default="/", help="where the node's file system starts (a staging directory for images)")
    ap.add_argument("--apply", action="store_true", help="write what differs (default: report only)")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--keys", default=None, help="file with the fleet's public ssh keys")
    a = ap.parse_args(argv)
    root = Path(a.root)
    items = desired(a.gpus, a.keys)
    facts = checks(a.gpus)
    changes = apply(items, root) if a.apply else diff(items, root)
    print(json.dumps({"root": str(root), "applied": bool(a.apply), "changes": changes, "checks": facts}, indent=1, default=str))
    if not all(f["ok"] for f in facts):
        return 2
    return 0 if (a.apply or not changes) else 1


if __name__ == "__main__":
    raise SystemExit(main())
