"""Destinations: values computed in place where they are going.

A concatenation whose pieces are each produced by one pointwise step and read by nothing else does not need its
pieces as tensors of their own: the result's storage is laid out first and every piece is computed straight into its
slice (the operator's ``out=`` form), after which the concatenation is a no-op.  That removes one pass over memory per
concatenation (rotary embeddings, gated halves, stacked projections).  The reference does the same at capture time:
``destined`` projects a gathered value's pieces into their parent's storage and ``views`` re-evaluates their aliases
from there, so that a result is computed in place in its destination (compiler/mesh_compiler/ir.py:185-274, the
``cat`` / zero ``pad`` cases at :243-254).

:func:`analyse` is the static part (which steps have a destination); the executor allocates and fills
(``runtime.Executor``, switch ``MESH_DESTINED``, on by default).
"""
from __future__ import annotations

import dataclasses
import os

import torch

from .ir import Plan, Ref
from .placement import POINTWISE, local_indices

aten = torch.ops.aten

# meta keys that make the executor treat a call specially (its operands or result are rewritten on the way)
_SPECIAL = ("draw", "causal_rows", "batch_arg", "bias_sizes", "groups_local", "once", "query_rows", "localize", "mean_as_sum", "vocab_parallel", "halo", "fallback")


def enabled() -> bool:
    return os.environ.get("MESH_DESTINED", "1") != "0"


@dataclasses.dataclass
class Destination:
    parent: str           # the concatenation's result
    at: int               # step index of the concatenation
    dim: int
    position: int         # which piece of the parent this value is
    pieces: tuple         # all piece names of the parent, in order


def _uses(plan: Plan) -> dict:
    count: dict[str, int] = {}

    def walk(o):
        if isinstance(o, Ref):
            count[o.name] = count.get(o.name, 0) + 1
        elif isinstance(o, (list, tuple)):
            for x in o:
                walk(x)
        elif isinstance(o, dict):
            for x in o.values():
                walk(x)
    for st in plan.steps:
        walk(st.args)
        walk(st.kwargs)
    for o in plan.outputs:
        if isinstance(o, str):
            count[o] = count.get(o, 0) + 1
    return count


def _has_out(target) -> bool:
    pkt = getattr(target, "overloadpacket", None)
    return pkt is not None and hasattr(pkt, "out")


def analyse(plan: Plan) -> dict[str, Destination]:
    """``{value name: Destination}`` for every value that can be computed into its concatenation's storage: all pieces
    of the concatenation are distinct results of pointwise calls (with an ``out=`` form, no special handling, a known
    cut and shape), read only by the concatenation, of the concatenation's own dtype."""
    uses = _uses(plan)
    producer = {st.out: (i, st) for i, st in enumerate(plan.steps)}
    found: dict[str, Destination] = {}
    for at, st in enumerate(plan.steps):
        if st.op != "call" or st.target is not aten.cat.default or not st.args or not isinstance(st.args[0], (list, tuple)):
            continue
        pieces = st.args[0]
        if len(pieces) < 2 or not all(isinstance(p, Ref) for p in pieces) or len({p.name for p in pieces}) != len(pieces):
            continue
        shape = plan.full_shapes.get(st.out)
        if shape is None:
            continue
        dim = (st.args[1] if len(st.args) > 1 else st.kwargs.get("dim", 0)) % max(1, len(shape))
        ok = True
        for p in pieces:
            i, src = producer.get(p.name, (None, None))
            if (src is None or i >= at or src.op != "call" or src.target not in POINTWISE or not _has_out(src.target)
                    or uses.get(p.name, 0) != 1 or any(k in src.meta for k in _SPECIAL)
                    or "out_specs" not in src.meta or "full_shape" not in src.meta
                    or plan.dtypes.get(p.name) != plan.dtypes.get(st.out)
                    or src.target in (aten.alias.default, aten.detach.default, aten.lift_fresh_copy.default)):
                ok = False
                break
        if not ok:
            continue
        names = tuple(p.name for p in pieces)
        for k, name in enumerate(names):
            found[name] = Destination(st.out, at, dim, k, names)
    return found


def local_shape(meta: dict, coords: tuple) -> tuple:
    """Shape of a step's result on the processor at ``coords``, from the cut the placement recorded for it."""
    shape = list(meta["full_shape"])
    for ax, s in enumerate(meta["out_specs"]):
        if getattr(s, "kind", "R") == "S" and len(shape) > s.dim:
            idx = local_indices(s, coords[ax], shape[s.dim])
            shape[s.dim] = len(range(*idx.indices(shape[s.dim]))) if isinstance(idx, slice) else len(idx)
    return tuple(shape)
