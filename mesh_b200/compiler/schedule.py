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
        "local_slices": sum(1 for s in plan.steps if s.op == "slice"),
        "levels": level,
        "uncovered": uncovered, "unwaited": unwaited, "redundant": redundant,
        "signature": sig.digest,
    }
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
