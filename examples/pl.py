#!/usr/bin/env python3
"""Parallel-layers language model, inference: attention and FFN read the same normalised input and their outputs are
added with learned weights; rotary positions; logits soft-capped at 30.  Megatron placement over the projections
(the reference's examples/pl.py:95-97 states the same cut for its model of this family)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from common import arguments, execute


class Rotary(nn.Module):
    def __init__(self, head_dim, seq, base=1000.0):
        super().__init__()
        inv = base ** (-torch.arange(0, head_dim, 2).float() / head_dim)
        ang = torch.outer(torch.arange(seq).float(), inv)
        self.register_buffer("cos", ang.cos()[None, :, None, :], persistent=False)
        self.register_buffer("sin", ang.sin()[None, :, None, :], persistent=False)

    def forward(self, x):
        h = x.shape[-1] // 2
        a, b = x[..., :h], x[..., h:]
        return torch.cat([a * self.cos + b * self.sin, b * self.cos - a * self.sin], -1)


class Layer(nn.Module):
    def __init__(self, dim, heads, mult, seq):
        super().__init__()
        self.heads, self.hd = heads, dim // heads
        self.norm = nn.LayerNorm(dim)
        self.wq, self.wk, self.wv = (nn.Linear(dim, dim, bias=False) for _ in range(3))
        self.wo = nn.Linear(dim, dim, bias=False)
        self.w1 = nn.Linear(dim, mult * dim, bias=False)
        self.w2 = nn.Linear(mult * dim, dim, bias=False)
        self.rot = Rotary(self.hd, seq)
        self.mix = nn.Parameter(torch.tensor([1.0, 1.0]))

    def forward(self, x):
        B, T, D = x.shape
        h = self.norm(x)
        q, k, v = (w(h).view(B, T, self.heads, self.hd) for w in (self.wq, self.wk, self.wv))
        q, k = self.rot(q), self.rot(k)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        a = self.wo(a.transpose(1, 2).reshape(B, T, D))
        f = self.w2(F.gelu(self.w1(h)))
        return x + self.mix[0] * a + self.mix[1] * f


class LM(nn.Module):
    def __init__(self, vocab, dim, heads, mult, layers, seq):
        super().__init__()
        self.emb = nn.Embedding(vocab, dim)
        self.layers = nn.ModuleList(Layer(dim, heads, mult, seq) for _ in range(layers))
        self.head = nn.Linear(dim, vocab, bias=False)

    def forward(self, ids):
        x = self.emb(ids)
        for l in self.layers:
            x = l(x)
        return 30 * torch.tanh(self.head(x) / 30)


def placement(procs):
    def choose(node):
        if node.op != "placeholder":
            return None
        n = node.name
        if any(n.endswith(f"{k}_weight") for k in ("wq", "wk", "wv", "w1")):
            return (0, procs, None)
        if any(n.endswith(f"{k}_weight") for k in ("wo", "w2")):
            return (1, procs, None)
        return None
    return choose


def main(argv=None):
    args = arguments(__doc__, argv)
    torch.manual_seed(0)
    vocab, dim, heads, mult, layers, batch, seq = (128, 64, 4, 2, 2, 2, 16) if args.small else (8192, 2048, 16, 4, 4, 2, 1024)
    model = LM(vocab, dim, heads, mult, layers, seq).to(args.device).eval()
    ids = torch.randint(0, vocab, (batch, seq), device=args.device)
    return execute(model, (ids,), placement, args)


if __name__ == "__main__":
    main()
