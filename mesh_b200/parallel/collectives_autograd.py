"""Differentiable collectives over a torch.distributed group (any backend, incl. ``mesh``).

all-gather <-> reduce-scatter and all-reduce <-> identity are each other's adjoints; these are the
``broadcast`` / ``reduce`` transfer kinds of the reference's reshard
(compiler/mesh_compiler/placement.py:250-340, :812-834) as eager autograd functions.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        out = torch.empty((x.shape[0] * w, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size(ctx.group)
        out = torch.empty((g.shape[0] // w, *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        out = torch.empty((x.shape[0] // w, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size(ctx.group)
        out = torch.empty((g.shape[0] * w, *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def all_gather_seq(x, group=None):
    return _AllGather.apply(x, group)


def reduce_scatter_seq(x, group=None):
    return _ReduceScatter.apply(x, group)


def all_reduce_sum(x, group=None):
    return _AllReduce.apply(x, group)


def copy_to_tp(x, group=None):
    return _CopyToTP.apply(x, group)
