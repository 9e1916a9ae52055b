"""Heterogeneous load balancing: stage model, cost rows, coupled share solve, capacity repair, ragged rows.

The reference extracts communication-delimited stages from a scheduled program, turns supplied or
measured per-unit costs into linear cost rows, and solves for the shares that minimise the sum over
stages of the slowest rank's time, with the collective time charged at the largest share and per-rank
caps (compiler/mesh_compiler/shares.py:38-424; solver rdma/mesh-graph.c:2072).  Same model here over
the SPMD plan; the solver is the native dense simplex (csrc/graph/graph.cpp).
"""
from __future__ import annotations

import collections
import math
import time

import torch

from .. import graph
from ..runtime import allocate
from .ir import Plan, Ref, Scheduled

aten = torch.ops.aten


def _work(step, plan: Plan) -> float:
    """Rough operation count of one call step on FULL shapes (matmuls: 2mnk; everything else: elements)."""
    if step.op != "call":
        return 0.0
    shp = plan.full_shapes.get(step.out, ())
    n = float(math.prod(shp)) if shp else 1.0
    if step.target in (aten.mm.default, aten.bmm.default, aten.addmm.default):
        refs = [a for a in step.args if isinstance(a, Ref)]
        a_shape = plan.full_shapes.get(refs[-2].name, ())
        k = a_shape[-1] if a_shape else 1
        return 2.0 * n * k
    return n


def stages(scheduled: Scheduled, segment=None, units=None):
    """Levels delimited by collectives.  Each stage: ``{"work": {part: ops}, "comm": {part: bytes}}`` where a
    step's *part* is ``segment(step)`` (default: the submodule path it was traced from, or ``"model"``)."""
    plan = scheduled.plan
    seg = segment or (lambda st: st.meta.get("module") or "model")
    out = [{"work": collections.Counter(), "comm": collections.Counter()}]
    by_channel = {t.channel: t for t in plan.transfers}
    last_part = "model"
    for st in plan.steps:
        if st.op == "collective":
            tr = by_channel.get(st.meta.get("channel"))
            out[-1]["comm"][last_part] += tr.nbytes if tr else 0
            out.append({"work": collections.Counter(), "comm": collections.Counter()})
        elif st.op == "call":
            sharded = any(s.kind in ("S", "P") for s in st.meta.get("out_specs", ()))
            part = seg(st) if sharded else None
            w = _work(st, plan)
            if part is None:
                out[-1]["work"]["__fixed__"] += w
            else:
                out[-1]["work"][part] += w
                last_part = part
    return [s for s in out if s["work"] or s["comm"]]


def supplied(staged, processors, rates: dict):
    """Cost rows from supplied rates: ``rates[processor]`` = operations per second (or ``{"ops": r}``).
    Returns ``(parts, fixed[s][j], coef[s][j][p])``."""
    parts = sorted({p for st in staged for p in st["work"] if p != "__fixed__"})
    names = list(processors)
    fixed, coef = [], []
    for st in staged:
        frow, crow = [], []
        for name in names:
            r = rates[name]["ops"] if isinstance(rates[name], dict) else rates[name]
            frow.append(st["work"].get("__fixed__", 0.0) / r)
            # a part's work on rank j scales with rank j's share of that part, times the number of ranks
            # already folded in: work is counted on full shapes, a share x does x of it
            crow.append([st["work"].get(p, 0.0) / r for p in parts])
        fixed.append(frow)
        coef.append(crow)
    return parts, fixed, coef


def measured(program, args, staged, processors, repeats: int = 3):
    """Cost rows from an observed run: time the program, attribute the time to stages by their operation
    counts, and assume every rank has the speed of the observed one (refined online by ``Allocator``)."""
    t0 = time.perf_counter()
    for _ in range(repeats):
        program(*args)
    dt = (time.perf_counter() - t0) / repeats
    total = sum(sum(st["work"].values()) for st in staged) or 1.0
    rate = total / dt
    return supplied(staged, processors, {name: rate for name in processors})


def solved(staged, costs, comm: float = 0.0, upper=None) -> dict:
    """``{part: ratios}`` minimising the summed stage times; ``comm`` = seconds per byte of collective traffic
    (the reference's default 1.0752e-10 s/byte is a Thunderbolt figure; NVLink 5 is ~1.3e-12)."""
    parts, fixed, coef = costs
    if not parts:
        return {}
    comm_rows = [[st["comm"].get(p, 0.0) * comm for p in parts] for st in staged]
    x, _ = graph.shares_coupled(fixed, coef, comm_rows, upper)
    return {p: tuple(x[i]) for i, p in enumerate(parts)}


def coupled(parts, comm, rows, upper):
    """Lower-level entry: ``rows`` = ``(stage, fixed_per_rank, {(part, rank): coefficient})`` like the reference's."""
    stages_n = 1 + max(r[0] for r in rows)
    ranks = len(upper)
    fixed = [[0.0] * ranks for _ in range(stages_n)]
    coef = [[[0.0] * len(parts) for _ in range(ranks)] for _ in range(stages_n)]
    idx = {p: i for i, p in enumerate(parts)}
    for s, fx, terms in rows:
        for j in range(ranks):
            fixed[s][j] += fx[j] if isinstance(fx, (list, tuple)) else fx
        for (p, j), c in terms.items():
            coef[s][j][idx[p]] += c
    comm_rows = [[st.get(p, 0.0) for p in parts] for st in comm] + [[0.0] * len(parts)] * (stages_n - len(comm))
    x, _ = graph.shares_coupled(fixed, coef, comm_rows, list(upper))
    return dict(zip(parts, (tuple(r) for r in x)))


def shifted(units, upper, load):
    """Greedy capacity repair on integer units: while some rank's fraction exceeds its cap, move one unit from
    the most over-full rank to the least loaded rank that still has room (shares.py:402-411)."""
    units = list(units)
    while True:
        total = sum(units)
        use = [u / total / cap for u, cap in zip(units, upper)]
        peak = max(range(len(units)), key=use.__getitem__)
        if use[peak] <= 1:
            return tuple(units)
        room = [j for j, cap in enumerate(upper) if (units[j] + 1) / total <= cap and j != peak]
        if not room:
            raise ValueError("shifted: the caps leave no room")
        units[min(room, key=lambda j: load(j, units))] += 1
        units[peak] -= 1


Ragged = collections.namedtuple("Ragged", "values offsets")


def rows(ragged: Ragged, speeds):
    """Partition a (possibly nested) ragged tensor's rows over ranks by speed: for every nesting level the row
    lengths and the cuts, innermost values last (shares.py:415-424)."""
    cuts = allocate.separators(ragged.offsets.tolist(), speeds)
    held = []
    while isinstance(ragged, Ragged):
        held.append((ragged.offsets.diff(), tuple(cuts)))
        cuts = ragged.offsets[torch.tensor(cuts)].tolist()
        ragged = ragged.values
    return (*held, (ragged, tuple(cuts)))
