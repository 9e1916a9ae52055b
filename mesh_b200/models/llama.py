"""Llama-style decoder blocks used by the compiler examples and tests.

The reference's canonical TP example is a 4-block Llama-style decoder (RMSNorm, causal multi-head
attention through SDPA, SwiGLU FFN) trained forward+backward with a scalar loss
(examples/parallel.py:25-75); this is the same model, parameterised.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight


class Block(nn.Module):
    def __init__(self, dim: int, heads: int, ffn: int):
        super().__init__()
        self.heads = heads
        self.attention_norm, self.ffn_norm = RMSNorm(dim), RMSNorm(dim)
        self.wq, self.wk, self.wv, self.wo = (nn.Linear(dim, dim, bias=False) for _ in range(4))
        self.w1, self.w3 = nn.Linear(dim, ffn, bias=False), nn.Linear(dim, ffn, bias=False)
        self.w2 = nn.Linear(ffn, dim, bias=False)

    def forward(self, x):
        B, T, D = x.shape
        h = self.attention_norm(x)
        q = self.wq(h).view(B, T, self.heads, -1).transpose(1, 2)
        k = self.wk(h).view(B, T, self.heads, -1).transpose(1, 2)
        v = self.wv(h).view(B, T, self.heads, -1).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, D)
        x = x + self.wo(a)
        h = self.ffn_norm(x)
        return x + self.w2(F.silu(self.w1(h)) * self.w3(h))


class Decoder(nn.Module):
    """``layers`` blocks and a squared-activation loss, like the reference's training example."""

    def __init__(self, dim: int = 256, heads: int = 4, ffn: int = 512, layers: int = 2):
        super().__init__()
        self.blocks = nn.ModuleList(Block(dim, heads, ffn) for _ in range(layers))

    def forward(self, x):
        for b in self.blocks:
            x = b(x)
        return x.float().pow(2).mean()


def megatron(processors, units=None):
    """The reference's Megatron placement (examples/parallel.py:77-89): ``wq, wk, wv, w1, w3`` split by output
    rows (column-parallel), ``wo, w2`` by input columns (row-parallel); ``units`` = optional share ratios."""
    names = tuple(processors)

    def placement(node):
        if node.op != "placeholder":
            return None
        n = node.name
        if any(f"_{k}_weight" in n or n.endswith(f"{k}_weight") for k in ("wq", "wk", "wv", "w1", "w3")):
            return (0, names, units)
        if any(f"_{k}_weight" in n or n.endswith(f"{k}_weight") for k in ("wo", "w2")):
            return (1, names, units)
        return None
    return placement


def data_parallel(processors, input_name: str = "x"):
    """Shard the batch dimension of the user input; parameters replicated -> gradient all-reduce."""
    names = tuple(processors)
    return lambda node: (0, names, None) if node.op == "placeholder" and node.name == input_name else None


def sequence_parallel(processors, input_name: str = "x", units=None, dim: int = 1):
    """Shard the sequence dimension of the input (``units="striped"`` for load-balanced causal attention)."""
    names = tuple(processors)
    return lambda node: (dim, names, units) if node.op == "placeholder" and node.name == input_name else None
