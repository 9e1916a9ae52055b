"""``python -m mesh_b200.tools.meshrun --nproc N [--max-restarts K] [--backoff S] -- script.py args...``

Launcher + supervisor for one node: starts one process per rank (each in its own process group) with the
torchrun environment (RANK, LOCAL_RANK, WORLD_SIZE, MASTER_ADDR=127.0.0.1, MASTER_PORT), watches them by
(pid, start time) identity, and when a rank exits without being asked: tells the survivors to stop (SIGTERM,
then a bounded wait — never SIGKILL while they may hold device state unless the wait runs out), and relaunches
the whole job, at most once per back-off interval, with ``MESH_RESTART=<n>`` so the script resumes from its last
checkpoint; with ``--shrink`` the job is re-formed at a smaller world, without the ranks that failed.  Signals to the supervisor: SIGHUP = restart the job, SIGUSR1 = release (stop the job, keep
supervising), SIGTERM = stop and exit — the reference's heartbeat supervisor (rdma/mesh-heartbeat.c:5-30, :135-325).
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time

from ..runtime.failure import alive, process_identity
from ..utils.launch import free_port

# A rank that ends because a PEER went away (a collective failed under it) exits with this code: the supervisor does
# not count it among the ranks that were lost when it re-forms the job at a smaller size.
PEER_LOST_EXIT = 75


class Supervisor:
    def __init__(self, cmd: list[str], nproc: int, max_restarts: int = 1, backoff_s: float = 60.0, grace_s: float = 20.0,
                 env: dict | None = None, log=None, shrink: bool = False, min_nproc: int = 1):
        self.cmd, self.nproc, self.max_restarts, self.backoff_s, self.grace_s = cmd, nproc, max_restarts, backoff_s, grace_s
        # shrink: the job is re-formed without the ranks that failed (their GPUs may be gone) instead of at the same
        # size; the script reads the new WORLD_SIZE and loads its sharded checkpoint re-cut for it
        self.shrink, self.min_nproc = shrink, max(1, min_nproc)
        self.env = dict(os.environ if env is None else env)
        self.procs: list[subprocess.Popen] = []
        self.ids: list[tuple] = []
        self.restarts = 0
        self.last_start = 0.0
        self.want = "run"
        self.log = log or (lambda **kw: print(json.dumps(kw), file=sys.stderr, flush=True))

    def launch(self) -> None:
        port = free_port()
        self.procs, self.ids = [], []
        for r in range(self.nproc):
            env = dict(self.env, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(self.nproc), MASTER_ADDR="127.0.0.1",
                       MASTER_PORT=str(port), MESH_RESTART=str(self.restarts))
            p = subprocess.Popen(self.cmd, env=env, start_new_session=True)
            self.procs.append(p)
            self.ids.append(process_identity(p.pid))
        self.last_start = time.monotonic()
        self.log(event="launched", nproc=self.nproc, restart=self.restarts, pids=[p.pid for p in self.procs])

    def stop_all(self) -> None:
        """Ask, wait (bounded), and only then force."""
        for p in self.procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
        deadline = time.monotonic() + self.grace_s
        for p in self.procs:
            try:
                p.wait(timeout=max(0.0, deadline - time.monotonic()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
                p.wait()

    def run(self) -> int:
        signal.signal(signal.SIGHUP, lambda *_: setattr(self, "want", "restart"))
        signal.signal(signal.SIGUSR1, lambda *_: setattr(self, "want", "release"))
        signal.signal(signal.SIGTERM, lambda *_: setattr(self, "want", "stop"))
        self.launch()
        while True:
            time.sleep(0.05)
            if self.want == "stop":
                self.stop_all()
                return 0
            if self.want == "release":
                self.stop_all()
                self.want = "idle"
            if self.want == "restart":
                self.stop_all()
                self.want = "run"
                self.launch()
                continue
            if self.want == "idle":
                continue
            codes = [p.poll() for p in self.procs]
            if all(c == 0 for c in codes):
                self.log(event="finished")
                return 0
            failed = [r for r, c in enumerate(codes) if c not in (None, 0)]
            gone = [r for r, (c, ident) in enumerate(zip(codes, self.ids)) if c is None and not alive(ident)]
            if failed or gone:
                self.log(event="rank_failed", ranks=failed + gone, codes=[codes[r] for r in failed])
                self.stop_all()
                if self.restarts >= self.max_restarts:
                    self.log(event="giving_up", restarts=self.restarts)
                    return 1
                wait = self.backoff_s - (time.monotonic() - self.last_start)
                if wait > 0:
                    time.sleep(wait)            # at most one reopen per back-off interval
                self.restarts += 1
                if self.shrink:
                    lost = [r for r in set(failed + gone) if codes[r] != PEER_LOST_EXIT]
                    smaller = self.nproc - max(1, len(lost))
                    if smaller < self.min_nproc:
                        self.log(event="giving_up", restarts=self.restarts, reason="fewer ranks left than --min-nproc")
                        return 1
                    self.nproc = smaller
                self.launch()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="meshrun")
    ap.add_argument("--nproc", type=int, required=True)
    ap.add_argument("--max-restarts", type=int, default=1)
    ap.add_argument("--backoff", type=float, default=60.0)
    ap.add_argument("--grace", type=float, default=20.0)
    ap.add_argument("--shrink", action="store_true", help="relaunch without the ranks that failed (a smaller world)")
    ap.add_argument("--min-nproc", type=int, default=1)
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.cmd[1:] if a.cmd and a.cmd[0] == "--" else a.cmd
    if not cmd:
        ap.error("no command given")
    if cmd[0].endswith(".py"):
        cmd = [sys.executable, *cmd]
    return Supervisor(cmd, a.nproc, a.max_restarts, a.backoff, a.grace, shrink=a.shrink, min_nproc=a.min_nproc).run()


if __name__ == "__main__":
    sys.exit(main())
