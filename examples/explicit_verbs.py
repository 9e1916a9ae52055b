"""A tensor-parallel FFN written with explicit parts and verbs instead of the compiler.

The reference's Swift examples (examples/indexed-gather.swift:17-40, examples/gram-chain.swift) drive the runtime this
way: the caller says where every tensor lives and which verb moves it; nothing is inferred.  Run on CPU ranks:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/explicit_verbs.py
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def build(world: int, tokens: int = 8, d: int = 16, ffn: int = 32, device="cpu"):
    from mesh_b200.distributed.program import Mesh
    m = Mesh(device=device)
    g = torch.Generator().manual_seed(0)
    w1 = torch.randn(d, ffn, generator=g) / d ** 0.5
    w2 = torch.randn(ffn, d, generator=g) / ffn ** 0.5
    cols = ffn // world
    x = m.tensor(on=0, sections=[(tokens, d)])[0]                                   # the activations start on rank 0
    xs = m.broadcast(x, to=range(world))
    up = [m.constant(r, w1[:, r * cols:(r + 1) * cols]) for r in range(world)]       # column-parallel
    down = [m.constant(r, w2[r * cols:(r + 1) * cols]) for r in range(world)]        # row-parallel
    partial = m.tensor(on=list(range(world)), sections=[(tokens, d)] * world)
    m.map(lambda a, u, v: torch.relu(a @ u) @ v, [[xs[r], up[r], down[r]] for r in range(world)],
          [[partial[r]] for r in range(world)], workers=range(world))
    y = m.reduce(partial, to=0)                                                      # the partial sums meet on rank 0
    return m.start(), x, y, (w1, w2)


def main() -> int:
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("gloo", rank=int(os.environ.get("RANK", 0)), world_size=int(os.environ.get("WORLD_SIZE", 1)))
    rank, world = dist.get_rank(), dist.get_world_size()
    m, x, y, (w1, w2) = build(world)
    worst = 0.0
    for i in range(3):
        inv = m.invocation(i)
        xv = torch.randn(8, 16, generator=torch.Generator().manual_seed(100 + i))
        if rank == 0:
            inv.part(x).copy_(xv)
        inv.submit()
        if rank == 0:
            worst = max(worst, float((inv.part(y) - torch.relu(xv @ w1) @ w2).abs().max()))
    if rank == 0:
        print({"ok": worst < 1e-4, "error": worst, "invocations": 3, "status": [m.result(i) for i in range(3)]})
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
