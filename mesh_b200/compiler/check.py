"""Static checks: the SPMD plan (definitions, collectives, channels) and the signal / wait protocols of the kernels.

Two checkers, both on the CPU and before anything runs on a GPU:

* :func:`check_plan` walks a compiled :class:`~mesh_b200.compiler.ir.Plan`: every value is defined once and before its
  use, every collective names an axis of the mesh with shard counts that fit the axis and the tensor, every inserted
  transfer has its own channel and a step that performs it, and the outputs exist.  The reference checks its plans'
  structure with a signature over the scheduled graph (compiler/mesh_compiler/schedule.py:58-134) and its buffers with
  a race check over strided views (rdma/mesh-graph.c); the view-level dependence analysis of this package lives in
  ``mesh_b200/csrc/graph/graph.cpp``.
* :func:`simulate` runs a model of kernels that signal and wait on monotonic counters (the protocol of every
  collective and fused kernel here: a launch raises counters on other ranks, waits until its own counters reach the
  values expected from the call sequence, then may raise more) and reports launches that can never finish.  Launches
  of a rank run in stream order.  :func:`collective_model` and :func:`exchange_model` state the protocols of
  ``collectives.cu`` in that form, so a sequence of calls can be proved free of deadlock for a given ring depth
  before it meets hardware, where a wrong expectation would only show as a bounded wait running out.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .ir import Plan, Ref


def _refs(obj, out: list) -> None:
    if isinstance(obj, Ref):
        out.append(obj.name)
    elif isinstance(obj, (tuple, list)):
        for o in obj:
            _refs(o, out)
    elif isinstance(obj, dict):
        for o in obj.values():
            _refs(o, out)


def check_plan(plan: Plan) -> list[str]:
    """Problems found in ``plan`` (empty list: none)."""
    problems: list[str] = []
    defined = set(plan.inputs)
    for name in plan.inputs:
        if name not in plan.input_specs:
            problems.append(f"input {name!r} has no sharding spec")
    seen_channels: dict[int, str] = {}
    by_value = {}
    for t in plan.transfers:
        if t.channel in seen_channels:
            problems.append(f"channel {t.channel} is used by transfers of {seen_channels[t.channel]!r} and {t.value!r}")
        seen_channels[t.channel] = t.value
        by_value.setdefault(t.value, []).append(t)
        if not 0 <= t.axis < len(plan.mesh.shape):
            problems.append(f"transfer of {t.value!r}: axis {t.axis} is not an axis of mesh {tuple(plan.mesh.shape)}")
    n_collective = 0
    for i, st in enumerate(plan.steps):
        used: list[str] = []
        _refs(st.args, used)
        _refs(st.kwargs, used)
        for u in used:
            if u not in defined:
                problems.append(f"step {i} ({st.op} -> {st.out!r}) uses {u!r} before it is defined")
        if st.out in defined:
            problems.append(f"step {i} defines {st.out!r} a second time")
        defined.add(st.out)
        if st.op == "fused" and "keep" in st.meta:
            defined.add(st.meta["keep"])                     # the gathered rows it hands on to the other readers
        if st.op == "fused" and "channel" in st.meta:
            n_collective += len(st.meta.get("channels", (st.meta["channel"],)))      # a fused step stands for its transfers
        if st.op == "collective":
            n_collective += 1
            ax = st.meta.get("axis")
            if ax is None or not 0 <= ax < len(plan.mesh.shape):
                problems.append(f"step {i}: collective on axis {ax!r}, mesh has {len(plan.mesh.shape)} axes")
                continue
            size = plan.mesh.shape[ax]
            for key in ("from", "to"):
                spec = st.meta.get(key)
                counts = getattr(spec, "counts", None)
                if counts:
                    if len(counts) != size:
                        problems.append(f"step {i}: {len(counts)} shard counts on an axis of {size} ranks")
                    full = plan.full_shapes.get(st.out)
                    dim = getattr(spec, "dim", None)
                    if full is not None and dim is not None and dim < len(full) and sum(counts) != full[dim]:
                        problems.append(f"step {i}: shard counts sum to {sum(counts)}, dimension {dim} of {st.out!r} is {full[dim]}")
    for o in plan.outputs:
        if isinstance(o, str) and o not in defined:
            problems.append(f"output {o!r} is never defined")
    if n_collective < len([t for t in plan.transfers if t.verb != "slice"]):
        problems.append(f"{len(plan.transfers)} transfers recorded but only {n_collective} collective steps")
    return problems


# --------------------------------------------------------------------------------------------- signal / wait model
@dataclass
class Launch:
    """One kernel launch: raise ``pre`` counters, wait until own counters reach ``waits``, then raise ``post``.
    Counters are named ``(rank, key)``; ``pre`` / ``post`` entries are ``(rank, key, add)``; ``waits`` are
    ``(key, value)`` on the launching rank's own counters."""
    name: str
    pre: list = field(default_factory=list)
    waits: list = field(default_factory=list)
    post: list = field(default_factory=list)


def simulate(programs: dict) -> list[str]:
    """Run the launches of every lane in order.  A key of ``programs`` is a rank, or ``(rank, lane)`` for parts of a
    rank's work that run concurrently (the sending and the receiving blocks of one exchange launch); counters belong
    to ranks.  Returns the launches that can never finish (empty: the sequence completes everywhere)."""
    rank_of = lambda k: k[0] if isinstance(k, tuple) else k
    counters: dict[tuple, int] = {}
    pc = {k: 0 for k in programs}
    started = {k: False for k in programs}
    progress = True
    while progress:
        progress = False
        for k, prog in programs.items():
            r = rank_of(k)
            while pc[k] < len(prog):
                ln = prog[pc[k]]
                if not started[k]:
                    for dst, key, add in ln.pre:
                        counters[(dst, key)] = counters.get((dst, key), 0) + add
                    started[k] = True
                    progress = True
                if all(counters.get((r, key), 0) >= value for key, value in ln.waits):
                    for dst, key, add in ln.post:
                        counters[(dst, key)] = counters.get((dst, key), 0) + add
                    pc[k] += 1
                    started[k] = False
                    progress = True
                else:
                    break
    stuck = []
    for k, prog in programs.items():
        if pc[k] < len(prog):
            r, ln = rank_of(k), prog[pc[k]]
            missing = [(w, v, counters.get((r, w), 0)) for w, v in ln.waits if counters.get((r, w), 0) < v]
            stuck.append(f"rank {r}: launch {pc[k]} {ln.name!r} waits for " +
                         ", ".join(f"{w} >= {v} (is {c})" for w, v, c in missing))
    return stuck


class CommModel:
    """Host-side bookkeeping of a communicator, as in ``distributed/comm.py``: parity of the staging buffer, expected
    counter totals, pieces sent and received per channel.  Every call appends to ``self.lanes``: lane ``"s"`` holds
    collectives and the sending blocks of exchanges, lane ``"r"`` the receiving blocks; a launch starts only when
    every part of the previous launch of the rank has finished (stream order)."""

    def __init__(self, rank: int, world: int, depth: int = 4, piece: int = 8 << 20):
        self.rank, self.world, self.depth, self.piece = rank, world, depth, piece
        self.turn = 0
        self.expect = [[0, 0], [0, 0]]
        self.sent = [0] * world
        self.rcvd = [0] * world
        self.lanes: dict[str, list[Launch]] = {"s": [], "r": []}
        self.calls = 0
        self.prev_parts = 0

    def programs(self) -> dict:
        return {(self.rank, lane): ls for lane, ls in self.lanes.items() if ls}

    def _open(self, name: str, lanes: list[str]) -> None:
        order = [(("done", self.calls - 1), self.prev_parts)] if self.calls else []
        for lane in lanes:
            self.lanes[lane].append(Launch(f"{name}/start", waits=list(order)))

    def _close(self, name: str, lanes: list[str]) -> None:
        for lane in lanes:
            self.lanes[lane].append(Launch(f"{name}/end", post=[(self.rank, ("done", self.calls), 1)]))
        self.prev_parts = len(lanes)
        self.calls += 1

    def collective(self, name: str, nblocks: int = 1, two_step: bool = False, waits_for=None, signals: bool = True) -> None:
        """publish -> wait -> pull (and a second round for the two-step all-reduce).  ``waits_for``: ranks this rank
        waits for (default all); ``signals=False``: a rank that only listens."""
        par = self.turn & 1
        self.turn += 1
        self.expect[par][0] += nblocks
        if two_step:
            self.expect[par][1] += nblocks
        ranks = range(self.world) if waits_for is None else waits_for
        self._open(name, ["s"])
        for step in range(2 if two_step else 1):
            pre = [(dst, ("arr", par, step, self.rank), nblocks) for dst in range(self.world)] if signals else []
            waits = [(("arr", par, step, src), self.expect[par][step]) for src in ranks]
            self.lanes["s"].append(Launch(f"{name}/{step}", pre=pre, waits=waits))
        self._close(name, ["s"])

    def exchange(self, name: str, nbytes: int, dsts=(), src=None, nb: int = 1) -> None:
        """The pull-based pipelined exchange: per piece the sender needs the ring slot free (acks of piece
        i - depth), stages and raises ``ready``; the receiver waits for ``ready``, pulls and raises ``ack``."""
        n = -(-nbytes // self.piece)
        lanes = (["s"] if dsts else []) + (["r"] if src is not None else [])
        if not lanes:
            return
        self._open(name, lanes)
        if dsts:
            base = {d: self.sent[d] for d in dsts}
            # every earlier message on the send channels has been pulled: the whole ring is free
            self.lanes["s"].append(Launch(f"{name}/drained", waits=[(("ack", d), base[d]) for d in dsts]))
            for i in range(n):
                waits = [(("ack", d), base[d] + (i - self.depth + 1) * nb) for d in dsts] if i >= self.depth else []
                self.lanes["s"].append(Launch(f"{name}/stage{i}", waits=waits, post=[(d, ("ready", self.rank), nb) for d in dsts]))
            for d in dsts:
                self.sent[d] += n * nb
        if src is not None:
            base = self.rcvd[src]
            for i in range(n):
                self.lanes["r"].append(Launch(f"{name}/pull{i}", waits=[(("ready", src), base + (i + 1) * nb)],
                                              post=[(src, ("ack", self.rank), nb)]))
            self.rcvd[src] += n * nb
        self._close(name, lanes)
