"""Schedule stage: dependence order, synchronisation signature, structure report, static sync check.

The plan that :mod:`placement` emits is already in a valid topological order of the exported graph.
This stage derives what the reference derives after placement (compiler/mesh_compiler/schedule.py:92-335;
rdma/mesh-graph.h:336-345; rdma/mesh_compile.py:8300-8355):

* the *declared transfers* (one per inserted collective) with their kind, consumer and weight;
* the *synchronisation signature*: the ordered list of operations at which processors wait for each
  other, which every processor must execute in the same order — the static check proves that each
  collective is entered by all members of its axis group with consistent sizes (``uncovered`` /
  ``unwaited`` / ``redundant`` counters);
* the *structure report*: ops absent from the plan, added copies, send/receive counts by collective kind;
* stage levels delimited by collectives (used by the share solver).
"""
from __future__ import annotations

import hashlib
from collections import Counter
from dataclasses import dataclass, field

from .ir import Plan, Ref, Step


def unit_cost(task) -> float:
    return 1.0


@dataclass
class Signature:
    operations: list          # (index, verb, kind, axis, value, nbytes)
    digest: str
    uncovered: int = 0        # reads of remote data not dominated by a wait
    unwaited: int = 0         # collectives whose result is never read
    redundant: int = 0        # back-to-back identical collectives on the same value
    levels: int = 0

    def ok(self) -> bool:
        return self.uncovered == 0


def _refs(obj, out):
    if isinstance(obj, Ref):
        out.append(obj.name)
    elif isinstance(obj, (list, tuple)):
        for x in obj:
            _refs(x, out)
    elif isinstance(obj, dict):
        for x in obj.values():
            _refs(x, out)


def schedule(plan: Plan, cost=unit_cost) -> tuple[Signature, dict]:
    """Returns ``(signature, structure)`` for a plan."""
    defined: dict[str, int] = {name: -1 for name in plan.inputs}
    used: Counter = Counter()
    ops = []
    uncovered = 0
    level = 0
    levels_of: dict[str, int] = {}
    seen_coll: dict[tuple, int] = {}
    redundant = 0
    for i, st in enumerate(plan.steps):
        refs: list[str] = []
        _refs(st.args, refs)
        _refs(st.kwargs, refs)
        for r in refs:
            if r not in defined:
                uncovered += 1            # a value read before any step (or wait) produced it
            used[r] += 1
        lvl = max([levels_of.get(r, 0) for r in refs], default=0)
        if st.op == "collective":
            m = st.meta
            key = (st.target, m["axis"], refs[0] if refs else None, repr(m["to"]))
            if key in seen_coll:
                redundant += 1
            seen_coll[key] = i
            nbytes = next((t.nbytes for t in plan.transfers if t.channel == m["channel"]), 0)
            ops.append((i, st.target, m["kind"], m["axis"], st.out, nbytes))
            lvl += 1
        levels_of[st.out] = lvl
        level = max(level, lvl)
        defined[st.out] = i
    for o in plan.outputs:
        if not isinstance(o, tuple):
            used[o] += 1
    unwaited = sum(1 for (_, _, _, _, name, _) in ops if used[name] == 0)
    h = hashlib.sha256()
    for (_, verb, kind, axis, _, nbytes) in ops:
        h.update(f"{verb}|{kind}|{axis}|{nbytes};".encode())
    sig = Signature(ops, h.hexdigest()[:16], uncovered, unwaited, redundant, level)
    by_kind = Counter(t.kind for t in plan.transfers)
    by_verb = Counter(t.verb for t in plan.transfers)
    structure = {
        "channels": len(plan.transfers),
        "by_kind": dict(by_kind),
        "by_verb": dict(by_verb),
        "bytes_between_processors": int(sum(t.nbytes for t in plan.transfers)),
        "calls": sum(1 for s in plan.steps if s.op == "call"),
        "fallbacks": sum(1 for s in plan.steps if s.meta.get("fallback")),
        # rule misses that cost something: an operand that was cut or partial had to be made whole first
        "gathering_fallbacks": sum(1 for s in plan.steps if s.meta.get("fallback") and s.meta.get("gathered")),
        "local_slices": sum(1 for s in plan.steps if s.op == "slice"),
        "levels": level,
        "uncovered": uncovered, "unwaited": unwaited, "redundant": redundant,
        "duplicated": getattr(plan, "duplicated", 0),
        "signature": sig.digest,
    }
    cp = copies(plan)
    structure["writes"] = len(cp.index)                    # distinct staged writes behind the transfers
    structure["shared_writes"] = len(plan.transfers) - len(cp.index) if plan.transfers else 0
    return sig, structure


def stages(plan: Plan) -> list[list[Step]]:
    """Communication-delimited levels (the stage model of the share solver, shares.py:38-90 of the reference)."""
    out: list[list[Step]] = [[]]
    for st in plan.steps:
        if st.op == "collective":
            out.append([])
        else:
            out[-1].append(st)
    return [s for s in out if s]


# ----------------------------------------------------------------------------- declared transfers, lifetimes, carried edges
@dataclass
class Declared:
    """One transfer of the plan with the steps that bound it in time (the reference's produced / read / consumed
    events of a declared transfer, compiler/mesh_compiler/schedule.py:198-284): the value it sends exists after step
    ``produced``, the transfer itself is step ``at``, its result is first read at ``read`` and last at ``consumed``
    (``len(steps)`` = a program output).  ``slack`` = steps between the producer and the transfer plus steps between
    the transfer and its first reader: what an overlapping executor can hide the transfer behind."""
    channel: int
    verb: str
    axis: int
    value: str
    result: str
    produced: int
    at: int
    read: int
    consumed: int
    nbytes: int
    weight: float = 1.0

    @property
    def slack(self) -> int:
        return max(0, self.at - self.produced - 1) + max(0, self.read - self.at - 1)


def _first_last_use(plan: Plan) -> tuple[dict, dict]:
    first: dict[str, int] = {}
    last: dict[str, int] = {}
    for i, st in enumerate(plan.steps):
        refs: list[str] = []
        _refs(st.args, refs)
        _refs(st.kwargs, refs)
        for r in refs:
            first.setdefault(r, i)
            last[r] = i
    end = len(plan.steps)
    for o in plan.outputs:
        if isinstance(o, str):
            first.setdefault(o, end)
            last[o] = end
    return first, last


def declarations(plan: Plan, cost=unit_cost) -> list[Declared]:
    """Every collective (plain or fused with its product) of the plan as a :class:`Declared` transfer."""
    produced = {name: -1 for name in plan.inputs}
    for i, st in enumerate(plan.steps):
        produced[st.out] = i
    first, last = _first_last_use(plan)
    by_channel = {t.channel: t for t in plan.transfers}
    out = []
    for i, st in enumerate(plan.steps):
        if not (st.op == "collective" or (st.op == "fused" and "channel" in st.meta)):
            continue
        m = st.meta
        src = st.args[0].name if st.args and isinstance(st.args[0], Ref) else st.out
        t = by_channel.get(m.get("channel"))
        out.append(Declared(m.get("channel", -1), st.target, m.get("axis", 0), src, st.out, produced.get(src, -1), i,
                            first.get(st.out, len(plan.steps)), last.get(st.out, len(plan.steps)),
                            t.nbytes if t is not None else 0, float(cost(st))))
    return out


def lifetimes(plan: Plan, itemsize=None) -> list[tuple[str, int, int, int]]:
    """``(value, first step, last step, bytes on one processor)`` for every value a step produces: what the
    workspace planner colours (values whose lifetimes do not overlap share bytes).  Sizes are those of the largest
    shard; ``itemsize(name)`` defaults to the plan's dtype table."""
    import math

    import torch
    _, last = _first_last_use(plan)
    out = []
    for i, st in enumerate(plan.steps):
        shape = plan.full_shapes.get(st.out)
        if shape is None:
            continue
        n = int(math.prod(shape)) if len(shape) else 1
        specs = plan.output_specs.get(st.out) if hasattr(plan, "output_specs") else None
        for s in (specs or ()):
            if getattr(s, "kind", "R") == "S" and s.counts and shape[s.dim]:
                n = n // shape[s.dim] * max(s.counts)
        dt = plan.dtypes.get(st.out, torch.float32)
        size = itemsize(st.out) if itemsize is not None else torch.empty((), dtype=dt).element_size() if isinstance(dt, torch.dtype) else 4
        out.append((st.out, i, max(i, last.get(st.out, i)), n * size))
    return out


def carried(plan: Plan, copies: int = 1) -> list[tuple[str, str, int]]:
    """Loop-carried dependences between successive executions of a standing plan: ``(earlier, later, lag)`` means the
    step ``later`` of execution ``t + lag`` must follow the step ``earlier`` of execution ``t``.  With ``copies`` sets
    of buffers, execution ``t + copies`` rewrites what execution ``t`` used: its first write of every input waits for
    the last read of that input ``copies`` executions earlier (write after read), and a collective's staging is
    reused by the same collective one execution later (lag 1: the sequence of collectives is the same in every
    execution, which is what lets their counters only grow).  The reference derives the same edges for its
    ``copies`` buffers (compiler/mesh_compiler/schedule.py:112-140, rdma/mesh-collective.c:390)."""
    first, last = _first_last_use(plan)
    edges = []
    for name in plan.inputs:
        if name in last:
            edges.append((f"read:{name}@{last[name]}", f"write:{name}", max(1, copies)))
    for d in declarations(plan):
        edges.append((f"{d.verb}:{d.result}@{d.at}", f"{d.verb}:{d.result}@{d.at}", 1))
    return edges


def horizon(plan: Plan, copies: int) -> int:
    """How many executions may be in flight at once: with ``copies`` input sets, execution ``t + copies`` may not
    start writing its inputs before execution ``t`` has read them, so at most ``copies`` executions overlap; a plan
    with no input at all (constants only) is bounded by its collectives' lag-1 edges, which stream order satisfies."""
    return max(1, copies)


# ----------------------------------------------------------------------------- copies: transfers that share one write
@dataclass
class Copies:
    """Transfers grouped by what they send: ``group[channel]`` is the key of a transfer (the value it sends, on which
    axis and in which form it leaves), ``index[key]`` numbers the distinct keys in plan order, ``member[k]`` lists the
    channels that share write ``k``.  Every collective here first copies its operand into this rank's staging buffer
    (publish, then the readers pull): transfers in one group publish the same bytes, so only the first member needs
    the copy and the later ones can raise their signals on it, provided nothing rewrote the staging slot in between
    (``reusable`` counts the members for which that holds: no other transfer on the same axis between them)."""
    group: dict
    index: dict
    member: dict
    reusable: int = 0


def copies(plan: Plan) -> Copies:
    """The logical copies of a plan's declared transfers (the reference groups its SENDs the same way before planning:
    each distinct (source, wire value, sent view, writers) is one write of its members,
    compiler/mesh_compiler/lower_inductor.py:7-32)."""
    produced = {}
    for i, st in enumerate(plan.steps):
        produced[st.out] = i
    group, order = {}, []
    for d in declarations(plan):
        st = plan.steps[d.at]
        # what leaves: the value, the axis it travels on, the verb's sending form (a gather and a broadcast of one value
        # both publish the whole local block; a scatter or an all-to-all publishes it cut for its readers)
        form = "cut" if d.verb in ("scatter", "all_to_all", "reduce_scatter", "mm_rs") else "whole"
        key = (d.value, d.axis, form, produced.get(d.value, -1))
        group[d.channel] = key
        order.append((d.at, d.channel, d.axis, key))
    index = {key: k for k, key in enumerate(dict.fromkeys(group.values()))}
    member: dict[int, list] = {}
    for ch, key in group.items():
        member.setdefault(index[key], []).append(ch)
    reusable = 0
    last_on_axis: dict[int, tuple] = {}
    for _, ch, axis, key in sorted(order):
        if last_on_axis.get(axis) == key:
            reusable += 1
        last_on_axis[axis] = key
    return Copies(group, index, member, reusable)


def planned(plan: Plan, step_us: float = 10.0, bucket_bytes: int = 32 << 20, staging_bytes: int = 64 << 20) -> dict:
    """The plan's declared transfers through the native planner (``runtime/plan.py::plan_transfers``): which transfers
    travel together as one demand, with which algorithm and in how many pieces, in which order on each axis, and how
    much of the link time the step cannot hide.  ``{"transfers": [declared + planned fields], "summary": {...}}``."""
    from ..runtime.plan import plan_transfers
    end = len(plan.steps)
    decl = declarations(plan)
    uses = {}
    for d in decl:
        uses[d.result] = d.read
    rows = [{"bytes": d.nbytes, "axis": d.axis, "verb": d.verb if d.verb in ("all_reduce", "all_gather", "reduce_scatter", "all_to_all")
             else {"ag_mm": "all_gather", "mm_rs": "reduce_scatter"}.get(d.verb, "point"),
             "at": d.at, "read": max(d.read, d.at), "groupable": d.verb == "all_reduce" and d.read >= end} for d in decl]
    out, summary = plan_transfers(rows, list(plan.mesh.shape), step_us=step_us, bucket_bytes=bucket_bytes,
                                  staging_bytes=staging_bytes) if rows else ([], {"link_us": 0.0, "exposed_us": 0.0,
                                                                                 "makespan_us": 0.0, "demands": 0})
    return {"transfers": [dict(channel=d.channel, verb=d.verb, value=d.value, result=d.result, **o) for d, o in zip(decl, out)],
            "summary": summary}


def pipelined(plan: Plan, cost=unit_cost, step_us: float = 10.0, observed: dict | None = None) -> dict:
    """The steady state of the plan when it is started again and again by an executor that overlaps transfers with
    compute (``runtime/plan.py::plan_pipeline``, the native planner's modulo scheduler): every step is a task - compute
    steps on the processor's stream in program order, every transfer on the links of its axis in program order, a
    transfer's duration from the planner's latency + bytes model, a compute step's from ``cost(step) * step_us`` - with
    the plan's data flow as dependences and the lag-1 edge of every collective (its staging is reused by the same
    collective of the next execution).  ``{"period_us", "latency_us", "copies", "resource_bound_us",
    "recurrence_bound_us", "bound_by"}``: how often an execution can start, how long one takes, how many sets of buffers
    that needs (what ``Prepared`` takes as its default ``copies``), and which resource sets the period.  ``observed``:
    a report of ``compiler/observe.py::observe`` for this plan - every step's measured time replaces its modelled one."""
    from ..runtime.plan import plan_pipeline
    steps = plan.steps
    n = len(steps)
    if n == 0:
        return {"period_us": 0.0, "latency_us": 0.0, "copies": 1, "resource_bound_us": 0.0, "recurrence_bound_us": 0.0,
                "bound_by": "nothing"}
    link_us = {}
    for t in planned(plan, step_us=step_us, bucket_bytes=0)["transfers"]:
        link_us[t["result"]] = max(0.0, t["end_us"] - t["start_us"])
    free = ("alias", "const", "slice")
    dur, res = [], []
    for st in steps:
        transfer = st.op == "collective" or (st.op == "fused" and "channel" in st.meta)
        if transfer:
            dur.append(link_us.get(st.out, step_us))
            res.append(1 + int(st.meta.get("axis", 0)))
        else:
            import operator
            nothing = st.op in free or st.target is operator.getitem
            dur.append(0.0 if nothing else float(cost(st)) * step_us)
            res.append(0)
    if observed is not None:
        for rec in observed.get("steps", ()):
            if 0 <= rec["index"] < n:
                dur[rec["index"]] = float(rec["seconds"]) * 1e6
    produced = {st.out: i for i, st in enumerate(steps)}
    edges, last_on = [], {}
    for i, st in enumerate(steps):
        refs: list[str] = []
        _refs(st.args, refs)
        _refs(st.kwargs, refs)
        for r in set(refs):
            if r in produced and produced[r] != i:
                edges.append((produced[r], i, 0))
        if res[i] in last_on:                              # a stream runs its tasks in program order
            edges.append((last_on[res[i]], i, 0))
        last_on[res[i]] = i
        if res[i] > 0:
            edges.append((i, i, 1))
    r = plan_pipeline(dur, res, edges)
    busy = {}
    for d, k in zip(dur, res):
        busy[k] = busy.get(k, 0.0) + d
    top = max(busy, key=busy.get)
    bound_by = "dependences" if r["recurrence_bound"] > r["resource_bound"] else ("compute" if top == 0 else f"links of axis {top - 1}")
    return {"period_us": r["period"], "latency_us": r["latency"], "copies": r["copies"], "resource_bound_us": r["resource_bound"],
            "recurrence_bound_us": r["recurrence_bound"], "bound_by": bound_by}
