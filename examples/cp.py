#!/usr/bin/env python3
"""Context-parallel causal language model: token ids, positions and targets are cut along the sequence, striped
(rank r holds tokens r, r + P, ...) so that causal attention work is balanced; the compiler evaluates the mask on
logical positions and moves K/V between the ranks.  Training loss and gradients against eager
(the reference's examples/cp.py:12-35 states this placement with ``units='striped'``)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from common import arguments, execute, units_of


class CausalLM(nn.Module):
    def __init__(self, vocab, dim, heads, seq):
        super().__init__()
        self.heads = heads
        self.tok, self.pos = nn.Embedding(vocab, dim), nn.Embedding(seq, dim)
        self.q, self.k, self.v, self.o = (nn.Linear(dim, dim, bias=False) for _ in range(4))
        self.head = nn.Linear(dim, vocab, bias=False)

    def forward(self, ids, positions, targets):
        x = self.tok(ids) + self.pos(positions)
        B, T, D = x.shape
        q, k, v = (w(x).view(B, T, self.heads, D // self.heads).transpose(1, 2) for w in (self.q, self.k, self.v))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, D)
        logits = self.head(x + self.o(a))
        return F.cross_entropy(logits.flatten(0, 1), targets.flatten())


def placement_for(units):
    def placement(procs):
        def choose(node):
            if node.op == "placeholder" and node.name in ("ids", "positions", "targets"):
                return (1, procs, units)
            return None
        return choose
    return placement


def main(argv=None):
    args = arguments(__doc__, argv)
    torch.manual_seed(0)
    vocab, dim, heads, batch, seq = (64, 32, 2, 2, 16) if args.small else (8192, 1024, 8, 1, 8192)
    model = CausalLM(vocab, dim, heads, seq).to(args.device)
    ids = torch.randint(0, vocab, (batch, seq), device=args.device)
    pos = torch.arange(seq, device=args.device)[None].expand(batch, seq).contiguous()
    tgt = torch.randint(0, vocab, (batch, seq), device=args.device)
    return execute(model, (ids, pos, tgt), placement_for(units_of(args) or "striped"), args, loss=0)


if __name__ == "__main__":
    main()
