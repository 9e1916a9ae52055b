"""Explicit collective verbs (functional API).

The reference's verbs are always stated by the caller, never inferred from how many peers there
are: send, gather, scatter, broadcast, all-gather, all-to-all, reduce, reduce-scatter, all-reduce,
with sum / max / min (design/collective-verbs.md:7-35; design/async-collectives.md:11-33).  These
functions are that surface over either a ``torch.distributed`` group (any backend, including
``mesh`` and gloo on CPU) or, for CUDA tensors when the process has a mesh context, directly over
the :class:`~mesh_b200.distributed.comm.Communicator`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .context import current_or_none

_RED = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "prod": dist.ReduceOp.PRODUCT,
        "avg": dist.ReduceOp.AVG}

def _communicator(t: torch.Tensor):
    """The mesh Communicator for CUDA tensors of a process that called ``mesh_b200.distributed.init``."""
    ctx = current_or_none()
    if ctx is None or not t.is_cuda or not ctx.is_cuda:
        return None
    return ctx.comm


def world_size(group=None) -> int:
    ctx = current_or_none()
    if ctx is not None and group is None:
        return ctx.world
    return dist.get_world_size(group) if dist.is_initialized() else 1


def all_reduce(t: torch.Tensor, op: str = "sum", group=None) -> torch.Tensor:
    c = _communicator(t) if group is None else None
    if c is not None:
        return c.all_reduce(t, op)
    if world_size(group) > 1:
        dist.all_reduce(t, _RED[op], group=group)
    return t


def all_gather(t: torch.Tensor, dim: int = 0, counts: list[int] | None = None, group=None) -> torch.Tensor:
    """Concatenate every rank's ``t`` along ``dim``; ``counts[r]`` = rank r's size along ``dim``."""
    W = world_size(group)
    if W == 1:
        return t
    tt = t.movedim(dim, 0).contiguous()
    counts = counts or [tt.shape[0]] * W
    out = torch.empty((sum(counts), *tt.shape[1:]), dtype=t.dtype, device=t.device)
    row = tt[0].numel() if tt.shape[0] else (out[0].numel() if out.shape[0] else 1)
    c = _communicator(t) if group is None else None
    if c is not None:
        c.all_gather(out, tt, [n * row for n in counts])
    elif len(set(counts)) == 1:
        dist.all_gather_into_tensor(out, tt, group=group)
    else:
        # library back ends want equal blocks: pad every block to the largest, gather, keep each rank's own rows
        top = max(counts)
        padded = tt.new_zeros((top, *tt.shape[1:]))
        padded[: tt.shape[0]] = tt
        blocks = tt.new_empty((W * top, *tt.shape[1:]))
        dist.all_gather_into_tensor(blocks, padded, group=group)
        at = 0
        for r, n in enumerate(counts):
            out[at:at + n] = blocks[r * top:r * top + n]
            at += n
    return out.movedim(0, dim)


def reduce_scatter(t: torch.Tensor, dim: int = 0, op: str = "sum", counts: list[int] | None = None, group=None):
    """Reduce every rank's ``t`` elementwise and keep this rank's segment along ``dim``."""
    W = world_size(group)
    if W == 1:
        return t
    ctx = current_or_none()
    rank = ctx.rank if (ctx is not None and group is None) else dist.get_rank(group)
    tt = t.movedim(dim, 0).contiguous()
    counts = counts or [tt.shape[0] // W] * W
    row = tt[0].numel()
    out = torch.empty((counts[rank], *tt.shape[1:]), dtype=t.dtype, device=t.device)
    c = _communicator(t) if group is None else None
    if c is not None:
        c.reduce_scatter(out, tt, op, [n * row for n in counts])
    elif len(set(counts)) == 1:
        dist.reduce_scatter_tensor(out, tt, _RED[op], group=group)
    else:
        # unequal segments: pad each to the largest with the reduction's identity, reduce-scatter equal blocks, trim
        top = max(counts)
        fill = 0 if op == "sum" else (float("-inf") if op == "max" else float("inf"))
        if not tt.dtype.is_floating_point and op != "sum":
            fill = torch.iinfo(tt.dtype).min if op == "max" else torch.iinfo(tt.dtype).max
        blocks = tt.new_full((W * top, *tt.shape[1:]), fill)
        at = 0
        for r, n in enumerate(counts):
            blocks[r * top:r * top + n] = tt[at:at + n]
            at += n
        mine = tt.new_empty((top, *tt.shape[1:]))
        dist.reduce_scatter_tensor(mine, blocks, _RED[op], group=group)
        out.copy_(mine[: counts[rank]])
    return out.movedim(0, dim)


def all_to_all(t: torch.Tensor, in_splits: list[int] | None = None, out_splits: list[int] | None = None, group=None):
    """MPI_Alltoallv over dim 0 (rdma/mesh_compile.py:1571-1579)."""
    W = world_size(group)
    if W == 1:
        return t
    t = t.contiguous()
    n_out = sum(out_splits) if out_splits is not None else t.shape[0]
    out = torch.empty((n_out, *t.shape[1:]), dtype=t.dtype, device=t.device)
    c = _communicator(t) if group is None else None
    if c is not None:
        c.all_to_all(out, t, out_splits, in_splits)
    else:
        dist.all_to_all_single(out, t, out_splits, in_splits, group=group)
    return out


def broadcast(t: torch.Tensor, root: int = 0, group=None) -> torch.Tensor:
    c = _communicator(t) if group is None else None
    if c is not None:
        return c.broadcast(t, root)
    if world_size(group) > 1:
        dist.broadcast(t, root, group=group)
    return t


def reduce(t: torch.Tensor, root: int = 0, op: str = "sum", group=None) -> torch.Tensor:
    c = _communicator(t) if group is None else None
    if c is not None:
        return c.reduce(t, root, op)
    if world_size(group) > 1:
        dist.reduce(t, root, _RED[op], group=group)
    return t


def gather(t: torch.Tensor, root: int = 0, group=None):
    W = world_size(group)
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    parts = [torch.empty_like(t) for _ in range(W)] if rank == root else None
    if W == 1:
        return [t]
    dist.gather(t, parts, dst=root, group=group)
    return parts


def scatter(out: torch.Tensor, parts: list[torch.Tensor] | None, root: int = 0, group=None) -> torch.Tensor:
    if world_size(group) == 1:
        out.copy_(parts[0])
        return out
    dist.scatter(out, parts, src=root, group=group)
    return out


def send(t: torch.Tensor, dst: int, group=None) -> None:
    c = _communicator(t) if group is None else None
    if c is not None:
        c.send(t.contiguous(), dst)
    else:
        dist.send(t, dst, group=group)


def recv(t: torch.Tensor, src: int, group=None) -> torch.Tensor:
    c = _communicator(t) if group is None else None
    if c is not None:
        return c.recv(t, src)
    dist.recv(t, src, group=group)
    return t
