"""Data parallelism with gradient reduce-scatter overlapped with the backward pass.

The reference expresses DP as batch sharding whose joint graph leaves partial gradients that are reduced
(compiler/mesh_compiler/placement.py:692-696, :812-834).  Eagerly, that is: parameters are grouped into buckets
in reverse order of use; when the last gradient of a bucket has been accumulated (autograd post-accumulate hooks)
the bucket is reduce-scattered on a side stream by this package's collective kernels while the backward pass
keeps computing; ``finish()`` joins the side stream.  Each rank ends up with the summed gradient of its 1/P
slice of every bucket (what a sharded optimizer needs); ``all_reduce=True`` gathers the slices back so that
``p.grad`` holds the full averaged gradient like DistributedDataParallel.
"""
from __future__ import annotations

import torch

from ..distributed import verbs


class _Bucket:
    def __init__(self, params, world):
        self.params = params
        self.numel = sum(p.numel() for p in params)
        self.per = -(-self.numel // world)
        self.padded = self.per * world
        p0 = params[0]
        self.flat = torch.zeros(self.padded, dtype=p0.dtype, device=p0.device)
        self.shard = torch.zeros(self.per, dtype=p0.dtype, device=p0.device)
        self.pending = len(params)
        self.offsets = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += p.numel()


class DataParallel:
    """Wraps a module: ``loss.backward()`` then ``dp.finish()``; gradients are averaged over the group."""

    def __init__(self, module: torch.nn.Module, world: int, rank: int, group=None, bucket_bytes: int = 64 << 20,
                 all_reduce: bool = True, axis=None):
        """``axis``: the data-parallel :class:`~mesh_b200.parallel.topology.AxisContext` of a grid job; on CUDA its
        communicator (this package's collective kernels over the axis' ranks) moves the buckets.  Without it the verbs
        pick the job-wide communicator (``group is None``) or the ``torch.distributed`` group."""
        self.module, self.world, self.rank, self.group, self.all_reduce = module, world, rank, group, all_reduce
        self.axis = axis
        params = [p for p in module.parameters() if p.requires_grad]
        self.buckets: list[_Bucket] = []
        cur, size = [], 0
        for p in reversed(params):                       # gradients become ready roughly in reverse order of use
            cur.append(p)
            size += p.numel() * p.element_size()
            if size >= bucket_bytes:
                self.buckets.append(_Bucket(cur, world))
                cur, size = [], 0
        if cur:
            self.buckets.append(_Bucket(cur, world))
        self._where = {}
        for b in self.buckets:
            for i, p in enumerate(b.params):
                self._where[p] = (b, i)
                p.register_post_accumulate_grad_hook(self._hook)
        cuda = params[0].is_cuda
        self.side = torch.cuda.Stream() if cuda else None
        self.launched = []
        self.next_bucket = 0

    def _hook(self, p):
        b, i = self._where[p]
        b.flat[b.offsets[i]: b.offsets[i] + p.numel()].copy_(p.grad.reshape(-1))
        b.pending -= 1
        # buckets are reduced strictly in order so that every rank issues the same sequence of collectives
        while self.next_bucket < len(self.buckets) and self.buckets[self.next_bucket].pending == 0:
            self._reduce(self.buckets[self.next_bucket])
            self.next_bucket += 1

    def _own_comm(self, t):
        ax = self.axis
        if ax is not None and t.is_cuda and getattr(ax, "_heap", None) is not None:
            return ax.comm
        return None

    def reduce_scatter(self, flat: torch.Tensor) -> torch.Tensor:
        c = self._own_comm(flat)
        if c is not None:
            out = torch.empty(flat.numel() // self.world, dtype=flat.dtype, device=flat.device)
            return c.reduce_scatter(out, flat, "sum")
        return verbs.reduce_scatter(flat, 0, "sum", group=self.group)

    def all_gather(self, shard: torch.Tensor) -> torch.Tensor:
        c = self._own_comm(shard)
        if c is not None:
            out = torch.empty(shard.numel() * self.world, dtype=shard.dtype, device=shard.device)
            return c.all_gather(out, shard.contiguous())
        return verbs.all_gather(shard, 0, group=self.group)

    def _reduce(self, b: _Bucket):
        if self.world == 1:
            b.shard.copy_(b.flat[: b.per])
            return
        if self.side is not None:
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                b.shard = self.reduce_scatter(b.flat)
                b.flat.record_stream(self.side)
        else:
            b.shard = self.reduce_scatter(b.flat)
        self.launched.append(b)

    def finish(self):
        """Join the side stream; returns the list of ``(bucket params, averaged gradient shard)``."""
        if self.side is not None:
            torch.cuda.current_stream().wait_stream(self.side)
        out = []
        for b in self.buckets:
            b.shard = b.shard / self.world
            if self.all_reduce and self.world > 1:
                full = self.all_gather(b.shard)
                for p, off in zip(b.params, b.offsets):
                    p.grad.copy_(full[off: off + p.numel()].view_as(p))
            out.append((b.params, b.shard))
            b.pending = len(b.params)
        self.launched.clear()
        self.next_bucket = 0
        return out
