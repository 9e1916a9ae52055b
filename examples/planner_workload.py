#!/usr/bin/env python3
"""A tick loop with a routed-expert planner whose tensor-parallel split follows the ranks' measured speed.

Every tick, each agent's state vector is routed to one of 8 experts (argmax of a small router) and goes through that
expert's two-layer FFN.  The experts' hidden columns are divided between the ranks: a rank applies its block of every
expert's up projection and the same rows of the down projection, so its output is a partial sum that one all-reduce
completes.  The operand's last row carries each rank's own segment time in its own column, so the same all-reduce hands
every rank every rank's time; an :class:`~mesh_b200.runtime.allocate.Allocator` (recursive least squares on
``t = a + b * columns``), stepped identically everywhere, sets the next tick's split.  This is the workload of the
reference's game planner (xonotic/planner/plan.py:21-75) without the game: ranks here are threads, or torchrun ranks,
and ``--slow`` makes some ranks artificially slower to show the split moving.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

EXPERTS, TEAMS = 8, 5


def model(width: int, ff: int):
    g = torch.Generator().manual_seed(20260828)
    mk = lambda *shape: torch.randn(*shape, generator=g) / shape[-2] ** 0.5
    return mk(width, EXPERTS), mk(EXPERTS, width, ff), mk(EXPERTS, ff, width), mk(width, TEAMS)


def solve(pos, route, up, down, out):
    """Rows grouped by expert (no per-row weight gather)."""
    sel = torch.argmax(pos @ route, 1)
    out.zero_()
    for e in range(EXPERTS):
        rows = (sel == e).nonzero().squeeze(1)
        if rows.numel():
            out[rows] = torch.relu(pos[rows] @ up[e]) @ down[e]


class ThreadAllReduce:
    """Sum over threads of one process (stand-in for the process group when the example runs without a launcher)."""

    def __init__(self, n):
        self.n, self.buf, self.bar = n, [None] * n, threading.Barrier(n)
        self.turn = threading.Lock()          # threads take turns computing, so that a segment's time is its own

    def __call__(self, rank, t):
        self.buf[rank] = t
        self.bar.wait()
        total = torch.stack(self.buf).sum(0)
        self.bar.wait()
        return total


def run_rank(rank, world, args, reduce, report):
    from mesh_b200.runtime.allocate import Allocator
    ff, width, bots = args.ff, args.width, args.bots
    grain = args.grain
    columns = [ff // world // grain * grain] * world
    columns[0] += ff - sum(columns)
    # prior per rank, in milliseconds: (a, b per column, var a = a^2, var b = (b/2)^2); floor = the least slope believed
    alloc = Allocator(columns, grain, [grain] * world, [(0.1, 2e-3, 1e-2, 1e-6)] * world, [1e-5] * world, forget=0.95, step=0.5)
    route, up, down, objective = model(width, ff)
    pos = torch.randn(bots, width, generator=torch.Generator().manual_seed(7)) * 0.1
    operand = torch.zeros(bots + 1, width)
    slow = args.slow[rank] if rank < len(args.slow) else 1.0
    history = []
    t_start = time.perf_counter()
    for tick in range(args.ticks):
        lo = sum(columns[:rank])
        hi = lo + columns[rank]
        with getattr(reduce, "turn", threading.Lock()):
            t0 = time.perf_counter()
            for _ in range(max(1, int(round(slow)))):      # a rank that is k times slower does its block k times
                solve(pos, route, up[:, :, lo:hi], down[:, lo:hi, :], operand[:bots])
            seg = time.perf_counter() - t0
        operand[bots].zero_()
        operand[bots, rank] = seg * 1e3                  # milliseconds
        total = reduce(rank, operand.clone())
        times = total[bots, :world].tolist()
        columns = alloc(times)
        history.append(max(times))
        # the plan: each agent's team objective from the completed expert output
        pos = pos + 0.01 * torch.tanh(total[:bots])
    if rank == 0:
        report.update({"ticks": args.ticks, "ranks": world, "columns": columns, "first_tick_ms": round(history[0], 4),
                       "last_tick_ms": round(sum(history[-5:]) / 5, 4), "ticks_per_s": round(args.ticks / (time.perf_counter() - t_start), 1),
                       "objective": [round(float(v), 4) for v in (pos @ objective).mean(0)]})


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--ticks", type=int, default=200)
    ap.add_argument("--bots", type=int, default=480)
    ap.add_argument("--width", type=int, default=256)
    ap.add_argument("--ff", type=int, default=2048)
    ap.add_argument("--grain", type=int, default=64)
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--slow", default="1,3", help="per-rank slowdown factors")
    args = ap.parse_args(argv)
    args.slow = [float(v) for v in args.slow.split(",")]
    torch.set_num_threads(1)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    report: dict = {}
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo")

        def reduce(rank, t):
            dist.all_reduce(t)
            return t
        run_rank(dist.get_rank(), world, args, reduce, report)
        dist.destroy_process_group()
    else:
        red = ThreadAllReduce(args.ranks)
        threads = [threading.Thread(target=run_rank, args=(r, args.ranks, args, red, report)) for r in range(args.ranks)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
    if report:
        print(json.dumps(report), flush=True)
    return report


if __name__ == "__main__":
    main()
