"""Run one command on all nodes, on all but this one, or on named nodes, each with a deadline, results streamed.

The reference's fleet tools (bin/mesh-run.sh: ``all | others | <name>``; bin/mesh-peers.sh: streaming and bounded by a
deadline; bin/mesh-status.sh) are shell over ssh.  This is the same interface for a multi-node job of this package:
nodes come from a hosts file (one ``name [address]`` per line, ``#`` comments) or ``--host`` flags, every node runs in
its own thread, a node that exceeds the deadline is reported as ``timeout`` and does not hold up the others, and each
result is printed as one JSON line as soon as it is there.

    python -m mesh_b200.tools.fleet run all -- nvidia-smi -L
    python -m mesh_b200.tools.fleet run others --hosts nodes.txt -- python -m mesh_b200.tools.runtime_id
    python -m mesh_b200.tools.fleet status                 # runtime identity of every node, and whether they agree
"""
from __future__ import annotations

import argparse
import json
import socket
import subprocess
import sys
import threading
import time
from pathlib import Path


def read_hosts(path) -> dict[str, str]:
    """``{name: address}`` from a hosts file (address defaults to the name)."""
    out = {}
    for line in Path(path).read_text().splitlines():
        line = line.split("#", 1)[0].strip()
        if line:
            parts = line.split()
            out[parts[0]] = parts[1] if len(parts) > 1 else parts[0]
    return out


def select(hosts: dict[str, str], which: str, me: str | None = None) -> dict[str, str]:
    me = me or socket.gethostname()
    if which == "all":
        return dict(hosts)
    if which == "others":
        return {n: a for n, a in hosts.items() if n != me and a != me}
    chosen = [w for w in which.split(",") if w]
    missing = [w for w in chosen if w not in hosts]
    if missing:
        raise KeyError(f"unknown node(s): {', '.join(missing)}")
    return {n: hosts[n] for n in chosen}


def ssh_runner(address: str, command: list[str], deadline_s: float) -> tuple[int, str, str]:
    local = address in ("localhost", "127.0.0.1", socket.gethostname())
    argv = command if local else ["ssh", "-o", "BatchMode=yes", "-o", "ConnectTimeout=10", address, *command]
    p = subprocess.run(argv, capture_output=True, text=True, timeout=deadline_s)
    return p.returncode, p.stdout, p.stderr


def run(hosts: dict[str, str], command: list[str], deadline_s: float = 60.0, runner=ssh_runner, emit=None) -> dict:
    """Run ``command`` on every node concurrently.  Returns ``{name: {"status", "code", "stdout", "stderr", "seconds"}}``
    with status ``ok`` / ``failed`` / ``timeout`` / ``error``; ``emit(name, record)`` is called as each node finishes."""
    results: dict = {}
    lock = threading.Lock()

    def one(name, address):
        t0 = time.monotonic()
        try:
            code, out, err = runner(address, command, deadline_s)
            rec = {"status": "ok" if code == 0 else "failed", "code": code, "stdout": out, "stderr": err}
        except subprocess.TimeoutExpired:
            rec = {"status": "timeout", "code": None, "stdout": "", "stderr": f"no answer within {deadline_s}s"}
        except Exception as e:
            rec = {"status": "error", "code": None, "stdout": "", "stderr": f"{type(e).__name__}: {e}"}
        rec["seconds"] = round(time.monotonic() - t0, 3)
        with lock:
            results[name] = rec
            if emit is not None:
                emit(name, rec)

    threads = [threading.Thread(target=one, args=(n, a), daemon=True) for n, a in hosts.items()]
    for t in threads:
        t.start()
    for t in threads:
        t.join(deadline_s + 5)
    for n in hosts:                                            # a runner that ignored its deadline
        results.setdefault(n, {"status": "timeout", "code": None, "stdout": "", "stderr": "runner did not return", "seconds": deadline_s})
    return results


def status(hosts: dict[str, str], deadline_s: float = 60.0, runner=ssh_runner) -> dict:
    """Every node's runtime identity (``tools/runtime_id.py``) and the keys on which the nodes differ."""
    from .runtime_id import same
    got = run(hosts, [sys.executable if len(hosts) == 1 else "python", "-m", "mesh_b200.tools.runtime_id"], deadline_s, runner)
    records, bad = {}, {}
    for n, r in got.items():
        try:
            records[n] = json.loads(r["stdout"]) if r["status"] == "ok" else None
        except ValueError:
            records[n] = None
        if records[n] is None:
            bad[n] = r["status"] if r["status"] != "ok" else "unreadable answer"
    alive = [r for r in records.values() if r is not None]
    return {"nodes": records, "unreachable": bad, "differ_on": same(alive) if len(alive) > 1 else []}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mesh-fleet")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("run", "status"):
        p = sub.add_parser(name)
        p.add_argument("--hosts", help="hosts file: one 'name [address]' per line")
        p.add_argument("--host", action="append", default=[], help="name or name=address; repeatable")
        p.add_argument("--deadline", type=float, default=60.0)
        if name == "run":
            p.add_argument("which", help="all | others | name[,name...]")
            p.add_argument("command", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    hosts = read_hosts(a.hosts) if a.hosts else {}
    for h in a.host:
        n, _, addr = h.partition("=")
        hosts[n] = addr or n
    if not hosts:
        hosts = {socket.gethostname(): "localhost"}
    if a.cmd == "status":
        rep = status(hosts, a.deadline)
        print(json.dumps(rep))
        return 0 if not rep["unreachable"] and not rep["differ_on"] else 1
    command = a.command[1:] if a.command[:1] == ["--"] else a.command
    if not command:
        ap.error("no command given")
    res = run(select(hosts, a.which), command, a.deadline,
              emit=lambda n, r: print(json.dumps({"node": n, **r}), flush=True))
    return 0 if all(r["status"] == "ok" for r in res.values()) else 1


if __name__ == "__main__":
    raise SystemExit(main())
