"""Sequence-parallel tensor-parallel SwiGLU FFN with stock NCCL collectives and cuBLAS GEMMs.

Model: the SwiGLU FFN of the reference's decoder block (examples/parallel.py:44-51) under its
``megatron()`` placement (:77-89): gate/up column-parallel, down row-parallel.  Collectives are the
ones its compiler would emit: all-gather before the column GEMMs, reduce-scatter after the row GEMM.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


class _AllGatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        out = torch.empty((x.shape[0] * world, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        world = dist.get_world_size(ctx.group)
        out = torch.empty((g.shape[0] // world, *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        out = torch.empty((x.shape[0] // world, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        world = dist.get_world_size(ctx.group)
        out = torch.empty((g.shape[0] * world, *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


def tp_ffn(x_shard, w_gate, w_up, w_down, group=None):
    """x_shard [M/P, D]; w_gate/w_up [F/P, D]; w_down [D, F/P] -> y shard [M/P, D]."""
    world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
    x = _AllGatherSeq.apply(x_shard, group) if world > 1 else x_shard
    h = F.silu(F.linear(x, w_gate)) * F.linear(x, w_up)
    y = F.linear(h, w_down)
    return _ReduceScatterSeq.apply(y, group) if world > 1 else y
