"""Explicit programs of parts, verbs and calls: declare once, start, submit invocations, read one status word each.

The reference's caller-facing model before its compiler existed (design/async-collectives.md:11-33, :136-147, :274-331;
design/collective-verbs.md:7-35; examples/indexed-gather.swift:17-40, examples/sync-on-remote-fill.swift:8-40) is a
``Mesh`` object on which the caller

* declares **parts** - tensors that live on one rank (``tensor(on:sections:)``, ``constant(on:bytes:)``),
* relates them with **explicit verbs** - ``send``, ``gather``, ``scatter``, ``broadcast``, ``allGather``, ``allToAll``,
  ``reduce``, ``reduceScatter``, ``allReduce`` - a verb is what the caller wrote, never inferred from how many peers
  happen to read a part; delivering the same immutable part to the same rank twice shares one receive,
* places **calls** of functions over parts on ranks (``call``, ``map``),
* then ``start()``s the program once and ``submit()``s invocations; each invocation ends in **one status word**
  (0, or an errno-style code), and ``syncOnRemoteFill`` exists but is explicit and never the default.

Here the same model runs on ``torch.distributed`` (gloo on CPU ranks, NCCL or this package's ``"mesh"`` backend on
GPUs).  Every rank builds the same program (it is deterministic), holds storage only for its own parts, and executes
the steps in program order; transfers of one verb go out as one batch of point-to-point operations.  Storage is kept
in ``copies`` sets, invocation ``i`` uses set ``i % copies``, so a caller may fill the inputs of the next invocation
while reading the results of the last.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Sequence

import torch
import torch.distributed as dist

from ..runtime.rendezvous import ECANCELED, ETIMEDOUT

_REDUCE = {"sum": lambda a, b: a + b, "max": torch.maximum, "min": torch.minimum}


@dataclasses.dataclass(frozen=True)
class Part:
    """A tensor that lives on one rank.  ``ident`` is its position in the program's table."""
    ident: int
    rank: int
    shape: tuple
    dtype: torch.dtype
    constant: bool = False


class Invocation:
    def __init__(self, program: "Mesh", index: int):
        self.program, self.index = program, index

    def submit(self) -> "Invocation":
        self.program._run(self.index)
        return self

    def part(self, part: Part) -> torch.Tensor:
        """This invocation's storage of ``part`` (only on the rank that owns it)."""
        return self.program.storage(part, self.index)


@dataclasses.dataclass(frozen=True)
class Placement:
    """Where transfers travel: ``routes[(source rank, destination rank)] = (relay, relay, ...)`` forces a delivery
    through the named ranks, in order, instead of the direct link (the reference lets the caller force relay paths the
    same way, ``Placement(routes:)``, examples/indexed-gather.swift:20-23; on a switch every pair has a direct link, so
    the default is no relay; a route is for shaping traffic or for machines that are not fully connected)."""
    routes: dict = dataclasses.field(default_factory=dict)

    def hops(self, src: int, dst: int) -> list[int]:
        via = [r for r in self.routes.get((src, dst), ()) if r not in (src, dst)]
        return via + [dst]


class Mesh:
    def __init__(self, rank: int | None = None, size: int | None = None, group=None, device="cpu", copies: int = 2,
                 placement: Placement | None = None):
        self.group = group
        self.placement = placement or Placement()
        self.rank = dist.get_rank(group) if rank is None else rank
        self.size = dist.get_world_size(group) if size is None else size
        self.device, self.copies = torch.device(device), copies
        self.parts: list[Part] = []
        self.steps: list[tuple] = []
        self.values: dict[int, torch.Tensor] = {}           # constants
        self.delivered: dict[tuple, Part] = {}              # (source part, destination rank) -> the copy there
        self.started = False
        self.store: list[dict[int, torch.Tensor]] = []
        self.status: dict[int, int] = {}
        self.cancelled = False

    # ------------------------------------------------------------------ declarations
    def _new(self, rank: int, shape, dtype, constant=False) -> Part:
        if self.started:
            raise RuntimeError("the program was started: declare everything before start()")
        if not 0 <= rank < self.size:
            raise ValueError(f"rank {rank} is not in a job of {self.size}")
        p = Part(len(self.parts), rank, tuple(shape), dtype, constant)
        self.parts.append(p)
        return p

    def tensor(self, on: int | Sequence[int], sections: Sequence[tuple], dtype=torch.float32):
        """One part per section on rank ``on`` (an int), or section ``i`` on rank ``on[i]`` (a sequence)."""
        ranks = [on] * len(sections) if isinstance(on, int) else list(on)
        if len(ranks) != len(sections):
            raise ValueError("one rank per section")
        return [self._new(r, s, dtype) for r, s in zip(ranks, sections)]

    def constant(self, on: int, value: torch.Tensor) -> Part:
        p = self._new(on, value.shape, value.dtype, constant=True)
        if on == self.rank:
            self.values[p.ident] = value.detach().to(self.device).clone()
        return p

    # ------------------------------------------------------------------ verbs
    def _deliver(self, part: Part, to: int) -> tuple[Part, list]:
        """The copy of ``part`` on rank ``to`` and the transfers that make it, hop by hop (none when it is there
        already).  A routed delivery lands on every relay first; a relay's copy is shared like any other."""
        if part.rank == to:
            return part, []
        origin = part.ident
        moves, here = [], part
        for hop in self.placement.hops(part.rank, to):
            if not 0 <= hop < self.size:
                raise ValueError(f"route through rank {hop}: not in a job of {self.size}")
            key = (origin, hop)
            if key in self.delivered:
                here = self.delivered[key]                  # the same immutable part: one receive is shared
                continue
            copy = self._new(hop, part.shape, part.dtype)
            self.delivered[key] = copy
            moves.append((here, copy))
            here = copy
        return here, moves

    def _transfers(self, pairs) -> list[Part]:
        """One verb: its direct transfers go out as one batch; relayed ones add a batch per further hop."""
        outs, by_depth = [], []
        for part, to in pairs:
            copy, moves = self._deliver(part, to)
            outs.append(copy)
            for depth, move in enumerate(moves):
                while len(by_depth) <= depth:
                    by_depth.append([])
                by_depth[depth].append(move)
        for moves in by_depth:
            self.steps.append(("move", moves))
        return outs

    def send(self, part: Part, to: int) -> Part:
        return self._transfers([(part, to)])[0]

    def gather(self, parts: Sequence[Part], to: int) -> list[Part]:
        return self._transfers([(p, to) for p in parts])

    def scatter(self, parts: Sequence[Part], to: Sequence[int]) -> list[Part]:
        if len(parts) != len(to):
            raise ValueError("one destination per part")
        return self._transfers(list(zip(parts, to)))

    def broadcast(self, part: Part, to: Sequence[int]) -> list[Part]:
        return self._transfers([(part, r) for r in to])

    def all_gather(self, parts: Sequence[Part]) -> dict[int, list[Part]]:
        """Every owner of a part gets all of them: ``{rank: [copies in the order of parts]}``."""
        owners = sorted({p.rank for p in parts})
        flat = self._transfers([(p, r) for r in owners for p in parts])
        return {r: flat[i * len(parts):(i + 1) * len(parts)] for i, r in enumerate(owners)}

    def all_to_all(self, parts: Sequence[Sequence[Part]]) -> list[list[Part]]:
        """``parts[j][i]``: what rank j holds for rank i.  Returns ``out[i][j]``: the same, delivered to rank i."""
        n = len(parts)
        flat = self._transfers([(parts[j][i], i) for i in range(n) for j in range(n)])
        return [flat[i * n:(i + 1) * n] for i in range(n)]

    def reduce(self, parts: Sequence[Part], to: int, op: str = "sum") -> Part:
        if op not in _REDUCE:
            raise ValueError(f"reductions are sum, max, min; not {op!r}")
        there = self.gather(parts, to)
        out = self._new(to, parts[0].shape, parts[0].dtype)
        self.steps.append(("reduce", to, [p.ident for p in there], out.ident, op))
        return out

    def reduce_scatter(self, contributions: Sequence[Sequence[Part]], to: Sequence[int], op: str = "sum") -> list[Part]:
        """``contributions[j][i]``: rank j's contribution to the section that ``to[i]`` owns."""
        return [self.reduce([row[i] for row in contributions], owner, op) for i, owner in enumerate(to)]

    def all_reduce(self, parts: Sequence[Part], op: str = "sum") -> list[Part]:
        """Every part's owner gets the reduction of all parts."""
        return [self.reduce(parts, p.rank, op) for p in parts]

    def sync_on_remote_fill(self, parts: Sequence[Part]) -> None:
        """Make the producers of these delivered parts wait until the receivers hold them (an acknowledgement comes
        back).  Never implied by a verb: it costs a round trip and, placed between two ranks that both wait before
        they send, it deadlocks - which the bounded wait then reports as a time-out in the status word."""
        back = []
        for copy in parts:
            src = next((s for (s, to), c in self.delivered.items() if c.ident == copy.ident), None)
            if src is not None:
                back.append((copy.rank, self.parts[src].rank))
        if back:
            self.steps.append(("ack", sorted(set(back))))

    # ------------------------------------------------------------------ compute
    def call(self, fn: Callable, inputs: Sequence[Part], outputs: Sequence[Part], on: int) -> None:
        """``fn(*input tensors) -> output tensor(s)`` on rank ``on``; all parts must live there."""
        for p in list(inputs) + list(outputs):
            if p.rank != on:
                raise ValueError(f"part {p.ident} lives on rank {p.rank}, the call is on rank {on}: deliver it first")
        self.steps.append(("call", on, fn, [p.ident for p in inputs], [p.ident for p in outputs]))

    def map(self, fn: Callable, inputs: Sequence[Sequence[Part]], outputs: Sequence[Sequence[Part]], workers: Sequence[int]) -> None:
        """The same function on several ranks, each over its own parts (``inputs[k]``, ``outputs[k]`` on ``workers[k]``)."""
        for k, w in enumerate(workers):
            self.call(fn, inputs[k], outputs[k], w)

    # ------------------------------------------------------------------ running
    def start(self, wait_s: float = 30.0) -> "Mesh":
        """Freeze the program and allocate this rank's storage (``copies`` sets)."""
        if self.started:
            return self
        self.started, self.wait_s = True, wait_s
        for _ in range(self.copies):
            self.store.append({p.ident: torch.zeros(p.shape, dtype=p.dtype, device=self.device)
                               for p in self.parts if p.rank == self.rank and not p.constant})
        return self

    def storage(self, part: Part, invocation: int = 0) -> torch.Tensor:
        if part.rank != self.rank:
            raise ValueError(f"part {part.ident} lives on rank {part.rank}, this is rank {self.rank}")
        if part.constant:
            return self.values[part.ident]
        if not self.started:
            raise RuntimeError("start() the program first")
        return self.store[invocation % self.copies][part.ident]

    def invocation(self, index: int) -> Invocation:
        if not self.started:
            raise RuntimeError("start() the program first")
        return Invocation(self, index)

    def result(self, index: int) -> int | None:
        """The invocation's status word: 0, ``ETIMEDOUT``, ``ECANCELED``; ``None`` while it has not been submitted."""
        return self.status.get(index)

    def cancel(self) -> None:
        """Invocations submitted from now on end at once with ``ECANCELED``."""
        self.cancelled = True

    def _peer(self, r: int) -> int:
        return r if self.group is None else dist.get_global_rank(self.group, r)

    def _exchange(self, ops) -> bool:
        if not ops:
            return True
        from datetime import timedelta
        try:
            for w in dist.batch_isend_irecv(ops):
                if w.wait(timeout=timedelta(seconds=self.wait_s)) is False:
                    return False
        except RuntimeError:
            return False                                      # a peer that never came: the bounded wait ran out
        return True

    def _run(self, index: int) -> None:
        if self.cancelled:
            self.status[index] = ECANCELED
            return
        me = self.rank
        get = lambda ident: self.storage(self.parts[ident], index)
        for step in self.steps:
            kind = step[0]
            if kind == "move":
                ops = []
                for src, dst in step[1]:
                    if src.rank == me:
                        ops.append(dist.P2POp(dist.isend, get(src.ident).contiguous(), self._peer(dst.rank), group=self.group))
                    if dst.rank == me:
                        ops.append(dist.P2POp(dist.irecv, get(dst.ident), self._peer(src.rank), group=self.group))
                if not self._exchange(ops):
                    self.status[index] = ETIMEDOUT
                    return
            elif kind == "reduce":
                _, to, idents, out, op = step
                if to == me:
                    acc = get(idents[0]).clone()
                    for k in idents[1:]:
                        acc = _REDUCE[op](acc, get(k))
                    get(out).copy_(acc)
            elif kind == "call":
                _, on, fn, ins, outs = step
                if on == me:
                    got = fn(*[get(k) for k in ins])
                    got = got if isinstance(got, (tuple, list)) else (got,)
                    if len(got) != len(outs):
                        raise ValueError(f"the function returned {len(got)} values for {len(outs)} output parts")
                    for k, t in zip(outs, got):
                        get(k).copy_(t)
            elif kind == "ack":
                word = torch.zeros(1, device=self.device)
                ops = []
                for frm, to in step[1]:
                    if frm == me:
                        ops.append(dist.P2POp(dist.isend, word, self._peer(to), group=self.group))
                    if to == me:
                        ops.append(dist.P2POp(dist.irecv, torch.zeros(1, device=self.device), self._peer(frm), group=self.group))
                if not self._exchange(ops):
                    self.status[index] = ETIMEDOUT
                    return
        self.status[index] = 0
