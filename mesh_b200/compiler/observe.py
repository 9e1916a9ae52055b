"""Observed costs: run a compiled program with every step timed, and report where the time went.

``observe(program, *args)`` returns, for the chosen processor, one record per step (kind, target, module path the step
was traced from, seconds; device-synchronised on CUDA), plus totals per module and per kind (calls / collectives /
fused).  ``stage_costs`` folds the records into the stage model of the share solver: observed seconds per stage
replace the operation-count estimate, which is how the reference feeds measured unit times into its solver
(``Bound.observe``, compiler/mesh_compiler/native.py:1391-1416; shares.py:243-322; the per-node ``Timed`` interpreter
of examples/tp.py:103-116).
"""
from __future__ import annotations

import os
from collections import defaultdict


def observe(program, *args, rank: int = 0, repeats: int = 2, **kwargs) -> dict:
    """``program``: a :class:`~mesh_b200.compiler.runtime.Program`.  The first run warms up; the median of the
    following ``repeats`` is reported."""
    old = os.environ.get("MESH_OBSERVE")
    os.environ["MESH_OBSERVE"] = "1"
    try:
        runs = []
        for _ in range(repeats + 1):
            program(*args, **kwargs)
            ex = program.per_rank[rank][0] if getattr(program, "threads", False) else program.exec
            runs.append(dict(ex.times))
            if not getattr(program, "threads", False):
                ex.times.clear()
    finally:
        if old is None:
            os.environ.pop("MESH_OBSERVE", None)
        else:
            os.environ["MESH_OBSERVE"] = old
    runs = runs[1:]
    steps = program.plan.steps
    records = []
    for i, st in enumerate(steps):
        ts = sorted(r.get(i, 0.0) for r in runs)
        records.append({"index": i, "op": st.op, "target": str(getattr(st.target, "__name__", st.target)),
                        "module": st.meta.get("module", ""), "out": st.out, "seconds": ts[len(ts) // 2]})
    by_module, by_kind = defaultdict(float), defaultdict(float)
    for r in records:
        by_module[r["module"] or "<top>"] += r["seconds"]
        by_kind[r["op"]] += r["seconds"]
    return {"rank": rank, "steps": records, "by_module": dict(by_module), "by_kind": dict(by_kind),
            "total": sum(r["seconds"] for r in records)}


def stage_costs(report: dict, plan) -> list[dict]:
    """Observed seconds per communication-delimited stage: ``[{"stage", "compute_s", "collective_s", "steps"}]``."""
    out, cur = [], {"stage": 0, "compute_s": 0.0, "collective_s": 0.0, "steps": 0}
    for rec, st in zip(report["steps"], plan.steps):
        if st.op == "collective" or (st.op == "fused" and "channel" in st.meta):      # a fused norm is compute
            cur["collective_s"] += rec["seconds"]
            cur["steps"] += 1
            out.append(cur)
            cur = {"stage": len(out), "compute_s": 0.0, "collective_s": 0.0, "steps": 0}
        else:
            cur["compute_s"] += rec["seconds"]
            cur["steps"] += 1
    if cur["steps"]:
        out.append(cur)
    return out
