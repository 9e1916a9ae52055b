"""Application bundles: pack a directory with a manifest of content hashes, verify, unpack, push to nodes.

The reference deploys an application as a tarball pushed to every node over ssh, identified by content hashes so that
nodes can tell whether they run the same thing (bin/mesh-application.py:1-131, design/APPLICATION-DEPLOYMENT.md).  The
same here, for multi-node jobs of this package:

* :func:`pack` - a ``.tar.gz`` whose first member is ``MANIFEST.json``: every file's size and SHA-256 and one digest of
  the whole tree (paths and hashes, sorted), so two bundles with the same digest hold the same bytes;
* :func:`verify` - re-hash a bundle (or an unpacked directory) against its manifest;
* :func:`unpack` - extract after checking free space and refusing members that would leave the destination;
* :func:`push` - copy the bundle to each host and unpack it there; the transport is a function so that tests (and
  single-host runs) can use a local copy, the default builds ``scp`` / ``ssh`` command lines with a deadline each.

    python -m mesh_b200.tools.application pack ./app app.tar.gz
    python -m mesh_b200.tools.application push app.tar.gz /opt/app --host n1 --host n2
"""
from __future__ import annotations

import argparse
import hashlib
import io
import json
import os
import subprocess
import tarfile
from pathlib import Path

from ..utils.disk import room

MANIFEST = "MANIFEST.json"
SKIP_DIRS = {".git", "__pycache__", ".pytest_cache"}


def _sha(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def manifest(root) -> dict:
    """``{"files": {relative path: {"bytes", "sha256"}}, "digest": sha256 over the sorted (path, sha256) pairs}``."""
    root = Path(root)
    files = {}
    for dirpath, dirnames, filenames in os.walk(root):
        dirnames[:] = sorted(d for d in dirnames if d not in SKIP_DIRS)
        for name in sorted(filenames):
            p = Path(dirpath) / name
            rel = p.relative_to(root).as_posix()
            if rel == MANIFEST or p.is_symlink() or not p.is_file():
                continue
            files[rel] = {"bytes": p.stat().st_size, "sha256": _sha(p)}
    tree = hashlib.sha256()
    for rel in sorted(files):
        tree.update(f"{rel}\0{files[rel]['sha256']}\n".encode())
    return {"files": files, "digest": tree.hexdigest(), "total_bytes": sum(f["bytes"] for f in files.values())}


def pack(root, bundle) -> dict:
    """Write ``bundle`` (``.tar.gz``) from the directory ``root``; returns the manifest."""
    root, bundle = Path(root), Path(bundle)
    man = manifest(root)
    room(bundle.parent if str(bundle.parent) else ".", man["total_bytes"] + (1 << 20))
    tmp = bundle.with_suffix(bundle.suffix + ".tmp")
    with tarfile.open(tmp, "w:gz") as tar:
        data = json.dumps(man, indent=1, sort_keys=True).encode()
        info = tarfile.TarInfo(MANIFEST)
        info.size = len(data)
        tar.addfile(info, io.BytesIO(data))
        for rel in sorted(man["files"]):
            tar.add(root / rel, arcname=rel, recursive=False)
    os.replace(tmp, bundle)
    return man


def read_manifest(bundle) -> dict:
    with tarfile.open(bundle, "r:gz") as tar:
        first = tar.next()
        if first is None or first.name != MANIFEST:
            raise ValueError("not an application bundle: the first member is not the manifest")
        return json.loads(tar.extractfile(first).read())


def verify(target) -> list[str]:
    """Problems found (empty: everything matches).  ``target``: a bundle, or a directory that holds ``MANIFEST.json``."""
    target = Path(target)
    problems = []
    if target.is_dir():
        man = json.loads((target / MANIFEST).read_text())
        now = manifest(target)
        for rel, rec in man["files"].items():
            got = now["files"].get(rel)
            if got is None:
                problems.append(f"missing: {rel}")
            elif got["sha256"] != rec["sha256"]:
                problems.append(f"changed: {rel}")
        problems += [f"extra: {rel}" for rel in now["files"] if rel not in man["files"]]
        return problems
    man = read_manifest(target)
    seen = set()
    with tarfile.open(target, "r:gz") as tar:
        for member in tar:
            if member.name == MANIFEST or not member.isfile():
                continue
            rec = man["files"].get(member.name)
            if rec is None:
                problems.append(f"extra: {member.name}")
                continue
            seen.add(member.name)
            if hashlib.sha256(tar.extractfile(member).read()).hexdigest() != rec["sha256"]:
                problems.append(f"changed: {member.name}")
    problems += [f"missing: {rel}" for rel in man["files"] if rel not in seen]
    return problems


def unpack(bundle, dest) -> dict:
    """Extract ``bundle`` into ``dest`` (created if needed); the manifest is written there too."""
    dest = Path(dest)
    man = read_manifest(bundle)
    dest.mkdir(parents=True, exist_ok=True)
    room(dest, man["total_bytes"] + (1 << 20))
    base = dest.resolve()
    with tarfile.open(bundle, "r:gz") as tar:
        for member in tar:
            out = (dest / member.name).resolve()
            if not (member.isfile() or member.isdir()) or (base != out and base not in out.parents):
                raise ValueError(f"refusing member {member.name!r}: not a plain file inside the destination")
            if hasattr(tarfile, "data_filter"):
                tar.extract(member, dest, filter="data")
            else:
                tar.extract(member, dest)
    problems = verify(dest)
    if problems:
        raise ValueError("unpacked tree does not match its manifest: " + "; ".join(problems[:5]))
    return man


def ssh_transport(host: str, bundle: Path, dest: str, deadline_s: float = 120.0) -> None:
    """Copy with scp, unpack with this module on the far side.  Each command has its own deadline."""
    remote = f"{dest.rstrip('/')}.bundle.tar.gz"
    opts = ["-o", "BatchMode=yes", "-o", "ConnectTimeout=10"]
    subprocess.run(["scp", *opts, str(bundle), f"{host}:{remote}"], check=True, timeout=deadline_s)
    subprocess.run(["ssh", *opts, host, "python", "-m", "mesh_b200.tools.application", "unpack", remote, dest],
                   check=True, timeout=deadline_s)


def push(bundle, dest: str, hosts: list[str], transport=ssh_transport) -> dict:
    """Deliver ``bundle`` to ``dest`` on every host; returns ``{host: "ok" | error text}`` and never stops at the
    first failure (a node that is down is reported, the others still get the bundle)."""
    bundle = Path(bundle)
    digest = read_manifest(bundle)["digest"]
    out = {"digest": digest, "hosts": {}}
    for h in hosts:
        try:
            transport(h, bundle, dest)
            out["hosts"][h] = "ok"
        except Exception as e:
            out["hosts"][h] = f"{type(e).__name__}: {e}"
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mesh-application")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("pack"); p.add_argument("root"); p.add_argument("bundle")
    p = sub.add_parser("verify"); p.add_argument("target")
    p = sub.add_parser("unpack"); p.add_argument("bundle"); p.add_argument("dest")
    p = sub.add_parser("push"); p.add_argument("bundle"); p.add_argument("dest"); p.add_argument("--host", action="append", default=[])
    a = ap.parse_args(argv)
    if a.cmd == "pack":
        man = pack(a.root, a.bundle)
        print(json.dumps({"digest": man["digest"], "files": len(man["files"]), "bytes": man["total_bytes"]}))
    elif a.cmd == "verify":
        problems = verify(a.target)
        print(json.dumps({"ok": not problems, "problems": problems}))
        return 0 if not problems else 1
    elif a.cmd == "unpack":
        print(json.dumps({"digest": unpack(a.bundle, a.dest)["digest"]}))
    else:
        rep = push(a.bundle, a.dest, a.host)
        print(json.dumps(rep))
        return 0 if all(v == "ok" for v in rep["hosts"].values()) else 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
