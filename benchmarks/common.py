"""Shared timing and reporting for the benchmark scripts."""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def init():
    """Join the torchrun job (or run solo) with the NCCL group and this package's context."""
    from mesh_b200.distributed import init as mesh_init
    return mesh_init(backend="nccl")


def barrier(world: int) -> None:
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def time_steps(fn, steps: int, warmup: int, world: int, device, flush_l2: bool = True, inner: int = 1) -> float:
    """Mean milliseconds per call of ``fn``: CUDA events around each call (around ``inner`` back-to-back calls for
    operations so short that the host's launch path would be what is timed), an L2-sized write between timed
    regions (untimed), max over ranks."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if flush_l2 else None
    for _ in range(max(3, warmup)):
        fn()
    barrier(world)
    evs = []
    for _ in range(steps):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(inner):
            fn()
        e1.record()
        evs.append((e0, e1))
    barrier(world)
    ms = sum(a.elapsed_time(b) for a, b in evs) / steps / inner
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def emit(rank: int, record: dict) -> None:
    if rank == 0:
        print(json.dumps(record), flush=True)
