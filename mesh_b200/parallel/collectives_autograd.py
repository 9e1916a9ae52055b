"""Differentiable collectives over a torch.distributed group (any backend, incl. ``mesh``).

all-gather <-> reduce-scatter and all-reduce <-> identity are each other's adjoints; these are the
``broadcast`` / ``reduce`` transfer kinds of the reference's reshard
(compiler/mesh_compiler/placement.py:250-340, :812-834) as eager autograd functions.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _comm_of(group, t):
    """``group`` may be a torch.distributed group or an axis context (``parallel/topology.py``); CUDA tensors of an
    axis that has a symmetric heap go through this package's collective kernels."""
    if hasattr(group, "ranks") and hasattr(group, "world"):
        if t.is_cuda and group._heap is not None:
            return group.comm, None
        return None, group.group
    return None, group


def _world(group) -> int:
    if hasattr(group, "ranks") and hasattr(group, "world"):
        return group.world
    if not (dist.is_available() and dist.is_initialized()):
        return 1                                   # a single process: every collective is the identity
    return dist.get_world_size(group)


def _ag(out, x, group):
    comm, g = _comm_of(group, x)
    if comm is not None:
        comm.all_gather(out, x)
    else:
        dist.all_gather_into_tensor(out, x, group=g)


def _rs(out, x, group):
    comm, g = _comm_of(group, x)
    if comm is not None:
        comm.reduce_scatter(out, x)
    else:
        dist.reduce_scatter_tensor(out, x, group=g)


def _ar(x, group):
    comm, g = _comm_of(group, x)
    if comm is not None:
        comm.all_reduce(x)
    else:
        dist.all_reduce(x, group=g)


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = _world(group)
        out = torch.empty((x.shape[0] * w, *x.shape[1:]), dtype=x.dtype, device=x.device)
        _ag(out, x.contiguous(), group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = _world(ctx.group)
        out = torch.empty((g.shape[0] // w, *g.shape[1:]), dtype=g.dtype, device=g.device)
        _rs(out, g.contiguous(), ctx.group)
        return out, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = _world(group)
        out = torch.empty((x.shape[0] // w, *x.shape[1:]), dtype=x.dtype, device=x.device)
        _rs(out, x.contiguous(), group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = _world(ctx.group)
        out = torch.empty((g.shape[0] * w, *g.shape[1:]), dtype=g.dtype, device=g.device)
        _ag(out, g.contiguous(), ctx.group)
        return out, None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        y = x.clone()
        _ar(y, group)
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
        _ar(g, ctx.group)
        return g, None


def all_gather_seq(x, group=None):
    return _AllGather.apply(x, group)


def reduce_scatter_seq(x, group=None):
    return _ReduceScatter.apply(x, group)


def all_reduce_sum(x, group=None):
    return _AllReduce.apply(x, group)


def copy_to_tp(x, group=None):
    return _CopyToTP.apply(x, group)
