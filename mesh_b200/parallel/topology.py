"""Processor grid of a job: data x pipeline x context x tensor parallel axes, and a context per axis.

The reference names a multi-dimensional grid of processors in its placements (``dimension`` / ``processors`` as
tuples, compiler/mesh_compiler/placement.py:57-69) and leaves the axis bookkeeping to the example programs.  Here
the grid is explicit: ranks are numbered with the tensor-parallel axis fastest (TP partners are NVLink neighbours
and exchange the most bytes per step), then context, pipeline, data.  Every axis gives this rank an
:class:`AxisContext` — rank and size along the axis, a ``torch.distributed`` group (NCCL or gloo; pipeline
send/recv and the CPU paths) and, on CUDA, a group view of the symmetric heap with a communicator of this
package's own kernels on it — which is what the parallel layers take as their ``ctx``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

AXES = ("tp", "cp", "pp", "dp")          # fastest varying first


@dataclass(frozen=True)
class ParallelDims:
    dp: int = 1
    pp: int = 1
    cp: int = 1
    tp: int = 1

    @property
    def world(self) -> int:
        return self.dp * self.pp * self.cp * self.tp

    def size(self, axis: str) -> int:
        return getattr(self, axis)

    def coords(self, rank: int) -> dict[str, int]:
        out = {}
        for ax in AXES:
            n = self.size(ax)
            out[ax] = rank % n
            rank //= n
        return out

    def rank_of(self, **coords: int) -> int:
        rank, mul = 0, 1
        for ax in AXES:
            c = coords.get(ax, 0)
            if not 0 <= c < self.size(ax):
                raise ValueError(f"{ax}={c} outside 0..{self.size(ax) - 1}")
            rank += c * mul
            mul *= self.size(ax)
        return rank

    def axis_ranks(self, rank: int, axis: str) -> list[int]:
        """World ranks of the group along ``axis`` that contains ``rank`` (the other coordinates fixed)."""
        c = self.coords(rank)
        return [self.rank_of(**{**c, axis: i}) for i in range(self.size(axis))]

    def groups(self, axis: str) -> list[list[int]]:
        """Every group of ``axis``, in a fixed order that all ranks agree on."""
        seen, out = set(), []
        for r in range(self.world):
            g = self.axis_ranks(r, axis)
            if g[0] not in seen and r == g[0]:
                seen.add(g[0])
                out.append(g)
        return out

    @staticmethod
    def parse(text: str) -> "ParallelDims":
        """``"tp2cp2pp2"``, ``"dp8"``, ``"tp4 x dp2"`` ..."""
        import re
        found = {k: int(v) for k, v in re.findall(r"(dp|pp|cp|tp)\s*=?\s*(\d+)", text.lower())}
        return ParallelDims(**found)

    def __str__(self) -> str:
        parts = [f"{ax}{self.size(ax)}" for ax in ("tp", "cp", "pp", "dp") if self.size(ax) > 1]
        return "x".join(parts) or "solo"


class AxisContext:
    """One axis of the grid as seen by this rank; has the attributes the parallel layers read from a context."""

    def __init__(self, name: str, rank: int, ranks: list[int], device: torch.device, group, heap=None):
        self.name, self.ranks = name, ranks
        self.rank, self.world = ranks.index(rank), len(ranks)
        self.device, self.group = device, group
        self.group_back = None       # pipeline axis: a second group for the traffic that flows toward earlier stages
        self._heap, self._comm = heap, None

    @property
    def is_cuda(self) -> bool:
        return self.device.type == "cuda"

    @property
    def heap(self):
        if self._heap is None:
            raise RuntimeError(f"axis {self.name}: no symmetric heap (CPU ranks use the process group)")
        return self._heap

    @property
    def comm(self):
        """Communicator of this package's kernels over the axis' ranks.  Collective over the whole job when first
        used: every rank must touch the same axes' communicators in the same order."""
        if self._comm is None:
            from ..distributed.comm import Communicator
            self._comm = Communicator(self.heap, staging_bytes=32 << 20, p2p_slot_bytes=16 << 20)
        return self._comm

    def peer(self, offset: int) -> int:
        """World rank of the member ``offset`` places along the axis (wrapping)."""
        return self.ranks[(self.rank + offset) % self.world]

    @property
    def first(self) -> bool:
        return self.rank == 0

    @property
    def last(self) -> bool:
        return self.rank == self.world - 1


class ParallelContext:
    """All axes for this rank.  ``ctx`` is the job's :class:`MeshContext` (or ``None`` for a solo CPU process)."""

    def __init__(self, ctx, dims: ParallelDims):
        world = 1 if ctx is None else ctx.world
        rank = 0 if ctx is None else ctx.rank
        if dims.world != world:
            raise ValueError(f"grid {dims} has {dims.world} ranks, the job has {world}")
        self.ctx, self.dims, self.rank, self.world = ctx, dims, rank, world
        self.device = torch.device("cpu") if ctx is None else ctx.device
        self.coords = dims.coords(rank)
        use_heap = ctx is not None and self.device.type == "cuda" and world > 1
        self.axes: dict[str, AxisContext] = {}
        for ax in AXES:
            mine = dims.axis_ranks(rank, ax)
            group = None
            if world > 1 and dist.is_initialized():
                if dims.size(ax) == world:
                    group = dist.group.WORLD
                elif dims.size(ax) > 1:
                    # new_group is collective over the job: every rank creates every group, in the same order
                    for g in dims.groups(ax):
                        h = dist.new_group(g)
                        if g == mine:
                            group = h
            back = None
            if ax == "pp" and dims.size(ax) > 1 and world > 1 and dist.is_initialized():
                # Activations flow toward later stages and gradients toward earlier ones.  Each direction gets a group
                # (a communicator) of its own, so that its sends and receives are queued in the order in which the data
                # comes into being and neither direction ever waits behind the other (parallel/pp.py).
                for g in dims.groups(ax):
                    h = dist.new_group(g)
                    if g == mine:
                        back = h
            heap = None
            if use_heap and dims.size(ax) > 1:
                heap = ctx.heap if dims.size(ax) == world else ctx.heap.group(mine)
            self.axes[ax] = AxisContext(ax, rank, mine, self.device, group, heap)
            self.axes[ax].group_back = back

    def __getattr__(self, name):
        axes = self.__dict__.get("axes", {})
        if name in axes:
            return axes[name]
        raise AttributeError(name)

    def describe(self) -> str:
        c = self.coords
        return f"rank {self.rank}/{self.world} grid {self.dims} at " + " ".join(f"{a}={c[a]}" for a in ("dp", "pp", "cp", "tp"))
