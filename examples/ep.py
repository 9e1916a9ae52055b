#!/usr/bin/env python3
"""Expert-parallel mixture of experts in the GShard form: softmax router, top-k, capacity-limited slots assigned in
token order (one-hot cumulative sum), tokens scattered into a packed ``[experts, participants * slots, dim]`` tensor,
one batched SwiGLU over the experts, weighted gather back.  Tokens and experts are both cut along their first
dimension; between them the packed tensor changes its cut from participants to experts, which the compiler turns
into an all-to-all (the reference's examples/ep.py:15-85 is the model of this program).

The production path for this layer is not the compiler but the fused kernels of ``mesh_b200/parallel/moe.py``
(``benchmarks/moe_ep.py``), which need no capacity limit."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from common import arguments, execute


class MoE(nn.Module):
    def __init__(self, dim, ffn, experts, k, slots):
        super().__init__()
        self.E, self.k, self.C = experts, k, slots
        self.router = nn.Parameter(torch.randn(dim, experts) * 0.02)
        self.w1 = nn.Parameter(torch.randn(experts, dim, ffn) * 0.02)
        self.w3 = nn.Parameter(torch.randn(experts, dim, ffn) * 0.02)
        self.w2 = nn.Parameter(torch.randn(experts, ffn, dim) * 0.02)

    def forward(self, x):
        """``x [participants, tokens, dim]``: every participant routes its own tokens."""
        G, S, M = x.shape
        E, k, C = self.E, self.k, self.C
        probs = torch.softmax(x @ self.router, -1)
        w, ids = probs.topk(k, -1)                                        # [G, S, k]
        onehot = F.one_hot(ids, E).reshape(G, S * k, E)                   # choices in token order
        place = ((onehot.cumsum(1) * onehot).sum(-1) - 1).reshape(G, S, k)
        keep = place < C
        w = w * keep
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-9)
        slot = torch.where(keep, ids * C + place, torch.full_like(ids, E * C))
        dispatch = F.one_hot(slot, E * C + 1)[..., : E * C].to(x.dtype)   # [G, S, k, E*C]
        combine = (dispatch * w[..., None]).sum(2)                        # [G, S, E*C]
        dispatch = dispatch.sum(2)
        packed = torch.bmm(dispatch.transpose(1, 2), x)                   # [G, E*C, M], cut over participants
        packed = packed.reshape(G, E, C, M).permute(1, 0, 2, 3)           # [E, G, C, M]: re-cut over experts = all-to-all
        packed = packed.reshape(E, G * C, M)
        h = F.silu(torch.bmm(packed, self.w1)) * torch.bmm(packed, self.w3)
        y = torch.bmm(h, self.w2).reshape(E, G, C, M).permute(1, 0, 2, 3)  # [G, E, C, M]: back over participants
        return torch.bmm(combine, y.reshape(G, E * C, M))


def placement(procs):
    def choose(node):
        if node.op == "placeholder":
            if node.name == "x" or any(node.name.endswith(n) for n in ("w1", "w2", "w3")):
                return (0, procs, None)
            return None
        # the two permutes are where the packed tensor changes hands: state the cut that the consumer wants
        if node.op == "call_function" and node.target is torch.ops.aten.permute.default and len(node.meta["val"].shape) == 4:
            return (0, procs, None)
        return None
    return choose


def main(argv=None):
    args = arguments(__doc__, argv)
    torch.manual_seed(0)
    import os
    p = max(args.nodes, int(os.environ.get("WORLD_SIZE", "1")))
    dim, ffn, experts, k, rows = (32, 48, 4, 2, 16) if args.small else (1024, 2816, 8, 2, 2048)
    slots = max(1, rows * k * 5 // (4 * experts))
    model = MoE(dim, ffn, experts, k, slots).to(args.device).eval()
    x = torch.randn(p, rows, dim, device=args.device)
    return execute(model, (x,), placement, args, tol=1e-3)


if __name__ == "__main__":
    main()
