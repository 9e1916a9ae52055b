#!/usr/bin/env python3
"""A chain of all-reduces of a sharded value, optionally with a matmul + tanh between them: the shape of a decode step
that crosses the machine once or twice per layer (141 crossings = a 35-layer decoder).  The step is one function compiled
once and called CROSSINGS times (the reference's examples/crossing.py:14-50 measures the same chain)."""
import os

import torch

from common import arguments, execute

HIDDEN = int(os.environ.get("HIDDEN", "1536"))
CROSSINGS = int(os.environ.get("CROSSINGS", "141"))
OVERLAP = os.environ.get("OVERLAP", "0") == "1"


class Crossing(torch.nn.Module):
    def __init__(self, hidden):
        super().__init__()
        self.register_buffer("weight", torch.randn(hidden, hidden) / hidden ** 0.5)

    def forward(self, x, y):
        received = x.sum(0, keepdim=True).expand_as(x)          # sharded rows summed: an all-reduce
        return (torch.tanh(y @ self.weight.mT), received) if OVERLAP else (received, y)


class Chain(torch.nn.Module):
    def __init__(self, work, n):
        super().__init__()
        self.work, self.n = work, n

    def forward(self, x, y):
        for _ in range(self.n):
            x, y = self.work(x, y)
        return x, y


def placement(procs):
    def choose(node):
        if node.op == "placeholder" and node.name in ("x", "y"):
            return (0, procs, None)
        return None
    return choose


def main(argv=None):
    args = arguments(__doc__, argv)
    torch.manual_seed(0)
    hidden, n = (64, 5) if args.small else (HIDDEN, CROSSINGS)
    model = Chain(Crossing(hidden), n).to(args.device).eval()
    p = max(args.nodes, int(os.environ.get("WORLD_SIZE", "1")))
    x = torch.randn(p, hidden, device=args.device) / 4
    y = torch.randn(p, hidden, device=args.device) / 4
    return execute(model, (x, y), placement, args, functions={"work"}, tol=2e-3)


if __name__ == "__main__":
    main()
