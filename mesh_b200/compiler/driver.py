"""Pipeline driver: capture -> place -> schedule -> ``Scheduled`` (compiler/mesh_compiler/driver.py:22-120).

    scheduled = compile_module(module, args, processors, placement, loss=0)
    result = Program(scheduled)(*args)

``processors``: ``{name: (machine, device)}`` in rank order (``device`` = ``"cuda:i"`` or ``"cpu"``);
``placement``: the callable contract of :mod:`mesh_b200.compiler.placement`; ``mesh``: optional grid shape
for N-D placements.  Compilation is host-only and deterministic: every rank derives the same plan from
the same inputs, so nothing needs to be exchanged.
"""
from __future__ import annotations

import math

from . import export as _export
from .ir import Scheduled
from .placement import place
from .schedule import schedule, unit_cost


def compile_captured(exported, processors, placement, cost=unit_cost, mesh=None) -> Scheduled:
    plan = place(exported, processors, placement, mesh)
    sig, structure = schedule(plan, cost)
    stated = {}
    for node in exported.graph_module.graph.nodes:
        if node.op == "placeholder":
            stated[node.name] = repr(plan.input_specs.get(node.name))
    names = list(processors)
    return Scheduled(exported, plan, dict(processors), stated, sig, structure, output_processor=names[0], cost=None)


def compile_module(module, args, processors, placement, cost=unit_cost, planning=None, machine=None, mesh=None,
                   kwargs=None, **export_options) -> Scheduled:
    """Ahead-of-time compile of one module call.  ``loss=<flat output index>`` compiles forward+backward."""
    exported = _export.export(module, args, kwargs, **export_options)
    inner = _cuts_inner_dimension(exported, placement) if "inner_cuts" not in export_options else 0
    if inner:
        # an input cut along an inner leading dimension (the batch of a sequence-first layout, the tokens of several
        # samples): capture again with the linear layers' leading dimensions kept apart (inference) or merged with the
        # cut dimension outermost (training), or the cut would be lost at the first flattening view
        exported = _export.export(module, args, kwargs, inner_cuts=inner, **export_options)
    sch = compile_captured(exported, processors, placement, cost, mesh)
    if exported.training and "decompositions" not in export_options and _gathers_for_batch_statistics(sch):
        # a training-mode batch norm whose input is cut along the batch (or a spatial dimension) would gather it to get
        # the statistics of the whole batch: capture again with the norm stated as means and sums, which become partial
        # sums and two small all-reduces
        from .decompose import norms
        exported = _export.export(module, args, kwargs, decompositions=norms(), **export_options)
        sch = compile_captured(exported, processors, placement, cost, mesh)
    return sch


def _gathers_for_batch_statistics(sch) -> bool:
    import torch
    aten = torch.ops.aten
    batch_norms = (aten._native_batch_norm_legit_functional.default, aten._native_batch_norm_legit.default,
                   aten._native_batch_norm_legit.no_stats, aten.native_batch_norm.default)
    return any(st.target in batch_norms and st.meta.get("fallback") and st.meta.get("gathered") for st in sch.plan.steps)


def _cuts_inner_dimension(exported, placement) -> int:
    """Does the stated placement cut a user input of three or more dimensions along a dimension that is neither its
    last nor, once dimensions of size one are set aside, its first?  (A cut behind leading dimensions of size one is
    still the outermost factor of the merged rows, which the view rule describes.)"""
    if not callable(placement):
        return 0
    for node in exported.graph_module.graph.nodes:
        if node.op != "placeholder":
            continue
        val = node.meta.get("val")
        nd = getattr(val, "ndim", 0)
        indices = nd == 2 and not (val.dtype.is_floating_point or val.dtype.is_complex)     # token ids: an embedding adds
        if nd < 3 and not indices:                                                           # the feature dimension later
            continue
        try:
            stated = placement(node)
        except Exception:
            continue
        if stated is None:
            continue
        for item in (stated if isinstance(stated, list) else [stated]):
            first = item[0] if isinstance(item, tuple) and item else None
            dims = [first] if isinstance(first, int) else [d for d in first if isinstance(d, int)] if isinstance(first, (tuple, list)) else []
            for dim in dims:                                 # (the N-D form states one dimension per grid axis)
                if 0 < dim % nd < nd - (0 if indices else 1) and math.prod(val.shape[:dim % nd]) > 1:
                    return dim % nd                          # the cut dimension (truthy: never the first)
    return 0


def compile_program(program, args, functions, processors, placement, cost=unit_cost, planning=None, machine=None,
                    mesh=None, **export_options) -> Scheduled:
    """A program whose ``forward`` only calls the named ``functions`` (compiled once, called many times)."""
    exported, calls = _export.calls(program, args, functions, **export_options)
    sch = compile_captured(exported, processors, placement, cost, mesh)
    sch.structure["function_calls"] = calls
    from .calls import analyse
    sch.structure["call_analysis"] = analyse(exported, functions).summary()
    return sch


def compiled(scheduled: Scheduled) -> Scheduled:
    """Attach (recompute) the synchronisation signature (driver.py:118 of the reference)."""
    scheduled.signature, scheduled.structure = schedule(scheduled.plan)
    return scheduled
