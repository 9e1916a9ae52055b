#!/usr/bin/env python3
"""Layers placed on different processors, possibly of different kinds (a GPU and the host CPU, say): every layer
is a projection + RMSNorm followed by a GeGLU FFN; layer i lives on processor i mod n, so each edge between
consecutive layers becomes a point-to-point transfer, and the last layer's partitions are combined by adding or
concatenating.  This is pipeline placement in its plainest form (the reference places its layers on named engines the
same way, examples/engines.py:91-131).  ``--device cuda:0,cpu`` gives one processor per listed device."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from common import arguments, execute


class Layer(nn.Module):
    def __init__(self, k, n):
        super().__init__()
        self.proj = nn.Parameter(torch.randn(k, k) / k ** 0.5)
        self.gate = nn.Parameter(torch.randn(n, k) / k ** 0.5)
        self.up = nn.Parameter(torch.randn(n, k) / k ** 0.5)
        self.down = nn.Parameter(torch.randn(k, n) / n ** 0.5)

    def forward(self, x):
        h = F.rms_norm(F.linear(x, self.proj), (x.shape[-1],), eps=1e-6)
        return x + F.linear(F.gelu(F.linear(h, self.gate), approximate="tanh") * F.linear(h, self.up), self.down)


class Stack(nn.Module):
    def __init__(self, k, n, layers, combine):
        super().__init__()
        self.layers = nn.ModuleList(Layer(k, n) for _ in range(layers))
        self.combine = combine

    def forward(self, x):
        outs = []
        for l in self.layers:
            x = l(x)
            outs.append(x)
        return outs[-1] + outs[-2] if self.combine == "add" else torch.cat(outs[-2:], -1)


def placement(procs):
    def choose(node):
        stack = node.meta.get("nn_module_stack") or {}
        for qual in stack:                                   # 'layers.3' -> processor 3 mod n
            parts = str(qual).replace("L__self___", "").replace("_", ".").split(".")
            if "layers" in parts:
                i = parts.index("layers")
                if i + 1 < len(parts) and parts[i + 1].isdigit():
                    return procs[int(parts[i + 1]) % len(procs)]
        if node.op == "placeholder" and "layers_" in node.name:
            digits = node.name.split("layers_")[1].split("_")[0]
            if digits.isdigit():
                return procs[int(digits) % len(procs)]
        return None
    return choose


def main(argv=None):
    args = arguments(__doc__, argv)
    torch.manual_seed(0)
    rows, k, n, layers = (8, 32, 48, 4) if args.small else (1024, 3840, 3456, 4)
    devices = args.device.split(",")
    if len(devices) > 1:                                     # one processor per listed device
        import common
        common.processors = lambda a: {f"{d.replace(':', '')}_{i}": (0, d) for i, d in enumerate(devices)}
        args.device = devices[0]
    model = Stack(k, n, layers, "add").to(args.device).eval()
    x = torch.randn(rows, k, device=args.device)
    return execute(model, (x,), placement, args, tol=1e-3)


if __name__ == "__main__":
    main()
