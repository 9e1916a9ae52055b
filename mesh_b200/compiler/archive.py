"""Compiled-program archives: ``save(directory, scheduled)`` / ``load(directory)``.

"Serialized objects we can resume without re-compiling" (rdma/mesh_compile.py:8398-8400): an archive holds
``state.pt`` (state tensors of the capture), ``program.pt2`` (the exported graph, torch.export's own format) and
``scheduled.json`` (processors, mesh, stated placements, signature digest, structure) —
compiler/mesh_compiler/archive.py:24-83.  Loading re-runs the deterministic placement stage on the saved
graph, which reproduces the plan bit for bit and is checked against the saved signature digest.
"""
from __future__ import annotations

import json
import os
from pathlib import Path

import torch

from ..utils.disk import room
from .ir import O, R, S, Scheduled, Spec


def _spec_json(s: Spec):
    return {"kind": s.kind, "dim": s.dim, "counts": list(s.counts), "striped": s.striped, "owner": s.owner, "op": s.op}


def _spec_from(d) -> Spec:
    return Spec(d["kind"], d["dim"], tuple(d["counts"]), d["striped"], d["owner"], d["op"])


def save(directory, scheduled: Scheduled, exported_program=None) -> None:
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    ex = scheduled.exported
    state = {name: t for name, (_, t) in ex.state.items() if isinstance(t, torch.Tensor)}
    need = sum(t.numel() * t.element_size() for t in state.values()) + (1 << 20)
    room(d, need)                                   # refuse to write into a nearly full volume
    tmp = d / "state.pt.tmp"
    torch.save(state, tmp)
    os.replace(tmp, d / "state.pt")
    if ex.program is None:
        raise ValueError("this Scheduled was not produced by export(): nothing to archive")
    torch.export.save(ex.program, str(d / "program.pt2"))
    plan = scheduled.plan
    meta = {
        "processors": {k: list(v) for k, v in scheduled.processors.items()},
        "mesh": list(plan.mesh.shape),
        "input_specs": {k: [_spec_json(s) for s in v] for k, v in plan.input_specs.items()},
        "output_specs": {str(i): [_spec_json(s) for s in plan.output_specs[o]] for i, o in enumerate(plan.outputs)
                         if not isinstance(o, tuple) and o in plan.output_specs},
        "signature": scheduled.signature.digest if scheduled.signature else None,
        "structure": scheduled.structure,
        "output_processor": scheduled.output_processor,
        "training": ex.training,
        "tied": dict(ex.tied),
    }
    tmp = d / "scheduled.json.tmp"
    tmp.write_text(json.dumps(meta, indent=1, default=str))
    os.replace(tmp, d / "scheduled.json")


def load(directory) -> Scheduled:
    from .driver import compile_captured
    d = Path(directory)
    meta = json.loads((d / "scheduled.json").read_text())
    from .export import read
    exported = read(torch.export.load(str(d / "program.pt2")), training=bool(meta.get("training")))
    state = torch.load(d / "state.pt", weights_only=False)
    for name, t in state.items():                 # the archive's own copy of the state tensors
        if name in exported.state:
            exported.state[name] = (exported.state[name][0], t)
    exported.tied = dict(meta.get("tied") or {})
    by_name = {qual: t for qual, t in exported.state.values()}
    for name, (qual, _t) in list(exported.state.items()):     # names that share a tensor read one tensor again
        if qual in exported.tied and exported.tied[qual] in by_name:
            exported.state[name] = (qual, by_name[exported.tied[qual]])
    input_specs = {k: tuple(_spec_from(s) for s in v) for k, v in meta["input_specs"].items()}
    out_specs = {int(i): tuple(_spec_from(s) for s in v) for i, v in meta["output_specs"].items()}
    processors = {k: tuple(v) for k, v in meta["processors"].items()}

    def placement(node):            # replay the stated placements exactly
        return None
    from .placement import Propagator
    from .ir import Mesh
    from .schedule import schedule
    mesh = Mesh(tuple(processors), tuple(meta["mesh"]))
    stated = {k: v for k, v in input_specs.items() if any(s.kind != "R" for s in v)}
    for i, v in out_specs.items():
        stated[("output", i)] = v
    order = [n.name for n in exported.graph_module.graph.nodes if n.op == "placeholder"]
    plan = Propagator(exported.graph_module, mesh, stated).run(order)
    sig, structure = schedule(plan)
    if meta["signature"] is not None and sig.digest != meta["signature"]:
        raise RuntimeError(f"archive {d}: replayed plan has signature {sig.digest}, saved {meta['signature']}")
    return Scheduled(exported, plan, processors, {k: repr(v) for k, v in input_specs.items()}, sig, structure,
                     output_processor=meta.get("output_processor"))
