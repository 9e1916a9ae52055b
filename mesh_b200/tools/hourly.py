"""Scheduled health run: ``python -m mesh_b200.tools.hourly [--gpus N] [--out runs.jsonl]``.

Runs the package's main programs one after the other, each under its own deadline, and appends one JSON line per
program to a report: exit status, seconds, the program's own JSON result when it printed one, and the tail of its
output when it failed.  A program that overruns its deadline is ended by process group (never by name) and recorded as
``timeout``; the run carries on with the next program.  Meant for a timer (cron / systemd) on a machine that should
notice regressions by itself (the reference's hourly run on its live pair, rdma/mesh_hourly.py:1-36, :124-213)."""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]


def programs(gpus: int) -> list[dict]:
    py = sys.executable
    run = [py] if gpus <= 1 else [py, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1"]
    return [
        {"name": "cpu_tests", "cmd": [py, "-m", "pytest", "tests", "-q", "-x", "-m", "not gpu"], "deadline_s": 1800},
        {"name": "tp_ffn_period", "cmd": run + ["bench.py", "--gpus", str(gpus)], "deadline_s": 600},
        {"name": "example_parallel", "cmd": [py, "examples/parallel.py", "--small"], "deadline_s": 300},
        {"name": "planner_workload", "cmd": [py, "examples/planner_workload.py", "--ticks", "100"], "deadline_s": 300},
        {"name": "micro_workloads", "cmd": [py, "benchmarks/micro.py", "all", "--small"], "deadline_s": 300},
    ]


def run_one(prog: dict, cwd: Path = ROOT) -> dict:
    t0 = time.time()
    rec = {"name": prog["name"], "started": t0}
    try:
        p = subprocess.Popen(prog["cmd"], cwd=cwd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                             start_new_session=True)
    except OSError as e:
        rec.update(status="not started", error=str(e), seconds=0.0)
        return rec
    try:
        out, _ = p.communicate(timeout=prog["deadline_s"])
        rec["status"] = "ok" if p.returncode == 0 else f"exit {p.returncode}"
    except subprocess.TimeoutExpired:
        os.killpg(p.pid, signal.SIGTERM)                 # the program's own process group, by id
        try:
            out, _ = p.communicate(timeout=10)
        except subprocess.TimeoutExpired:
            os.killpg(p.pid, signal.SIGKILL)
            out, _ = p.communicate()
        rec["status"] = "timeout"
    rec["seconds"] = round(time.time() - t0, 2)
    for line in reversed((out or "").splitlines()):
        if line.startswith("{"):
            try:
                rec["result"] = json.loads(line)
                break
            except ValueError:
                pass
    if rec["status"] != "ok":
        rec["tail"] = (out or "")[-800:]
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mesh-hourly")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--out", default=str(ROOT / "hourly.jsonl"))
    ap.add_argument("--only", default=None, help="comma-separated program names")
    a = ap.parse_args(argv)
    from ..utils.disk import room
    progs = [p for p in programs(a.gpus) if a.only is None or p["name"] in a.only.split(",")]
    bad = 0
    for prog in progs:
        rec = run_one(prog)
        bad += rec["status"] != "ok"
        try:
            room(os.path.dirname(os.path.abspath(a.out)), 1 << 20)      # never fill the disk with reports
            with open(a.out, "a") as f:
                f.write(json.dumps(rec) + "\n")
        except OSError as e:
            print(json.dumps({"name": prog["name"], "report_not_written": str(e)}), flush=True)
        print(json.dumps({k: rec[k] for k in ("name", "status", "seconds")}), flush=True)
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
