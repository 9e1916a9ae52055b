"""Generated host programs: one Python function per processor that IS the program, not a description of it.

``lower`` prints what a processor will do and runs it through the interpreting executor.  ``generate`` goes one step
further, the way the reference generates the host program that encodes a lowered program's dispatches
(rdma/mesh_metal4.py: generator and runner): every plain operator call of the processor's steps becomes a line that
calls the operator directly on local variables, with no step table walked and no argument tree resolved at run time;
collectives, fused steps and the calls the executor treats specially (draws, attention over a row shard, localised
shapes, products that may run on this package's kernels) call the executor's method for that step.  The text is
self-contained Python (it can be stored beside an archive and read), ``HostProgram.load()`` turns it into a callable,
and running it gives the numbers of the interpreted plan.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .ir import Plan, Ref
from .lower import lower

aten = torch.ops.aten

# meta keys and targets that need the executor's own handling
_SPECIAL = ("draw", "causal_rows", "batch_arg", "bias_sizes", "groups_local", "once", "query_rows", "localize", "mean_as_sum", "vocab_parallel", "halo", "fallback")
_DISPATCHED = (aten.mm.default, aten.matmul.default, aten.scaled_dot_product_attention.default, aten.view.default,
               aten._unsafe_view.default)


def _lit(a) -> str | None:
    """Source text of an argument, or None when it cannot be written as a literal."""
    if isinstance(a, Ref):
        return a.name
    if isinstance(a, (list, tuple)):
        parts = [_lit(x) for x in a]
        if any(p is None for p in parts):
            return None
        inner = ", ".join(parts)
        return f"[{inner}]" if isinstance(a, list) else f"({inner}{',' if len(a) == 1 else ''})"
    if isinstance(a, torch.dtype):
        return str(a)
    if isinstance(a, torch.device):
        return "ex.device"
    if isinstance(a, torch.memory_format):
        return str(a)
    if isinstance(a, torch.layout):
        return str(a)
    if a is None or isinstance(a, (bool, int, str)):
        return repr(a)
    if isinstance(a, float):
        return repr(a) if a == a and abs(a) != float("inf") else f"float({str(a)!r})"
    return None


def _view(st, coords) -> str | None:
    """A view whose target shape is localised for this processor when the program is generated (the interpreter does
    it at every execution): ``x.reshape(shape)``."""
    m = st.meta
    if any(k in m for k in _SPECIAL if k != "localize") or len(st.args) != 2 or not isinstance(st.args[0], Ref):
        return None
    shape = list(st.args[1])
    if not all(isinstance(v, int) for v in shape):
        return None
    if "localize" in m and "out_specs" in m:
        full = m["full_shape"]
        for ax, sp in enumerate(m["out_specs"]):
            if getattr(sp, "kind", "R") == "S" and len(shape) == len(full):
                shape[sp.dim] = sp.counts[coords[ax]]
        if -1 in shape and len(shape) == len(full):
            shape = [full[k] if v == -1 else v for k, v in enumerate(shape)]
    x = st.args[0].name
    return f"None if {x} is None else {x}.reshape({shape!r})"


def _direct(st, coords=()) -> str | None:
    """``aten.<op>.<overload>(...)`` for a step that is a plain operator call, else None."""
    import operator
    t = st.target
    if t is operator.getitem and isinstance(st.args[0], Ref) and isinstance(st.args[1], int):
        x = st.args[0].name
        return f"None if {x} is None else {x}[{st.args[1]}]"
    if t in (aten.view.default, aten._unsafe_view.default):
        return _view(st, coords)
    if not isinstance(t, torch._ops.OpOverload) or t.namespace != "aten" or t in _DISPATCHED or any(k in st.meta for k in _SPECIAL):
        return None
    stated = list(st.meta.get("out_specs", ())) + [sp for item in st.meta.get("items", {}).values() for sp in item[0]]
    if any(getattr(sp, "kind", "R") == "S" and 0 in sp.counts for sp in stated):
        return None                               # some processor's share is empty: the executor states that result itself
    args = [_lit(a) for a in st.args]
    kwargs = {k: _lit(v) for k, v in st.kwargs.items()}
    if any(a is None for a in args) or any(v is None for v in kwargs.values()):
        return None
    if "device" in kwargs and st.kwargs["device"] is not None:
        kwargs["device"] = "ex.device"
    refs = sorted(set(_names(st)))
    call = f"aten.{t._schema.name.split('::')[1]}.{t._overloadname}({', '.join(args + [f'{k}={v}' for k, v in kwargs.items()])})"
    if refs:                                  # an operand that lives on another processor: the result does too
        return f"None if ({' or '.join(f'{r} is None' for r in refs)}) else {call}"
    return call


@dataclass
class HostProgram:
    name: str
    rank: int
    source: str
    steps: list                                # the plan's steps, indexed by the generated code
    direct: int = 0                            # lines that call an operator directly
    through_executor: int = 0                  # lines that call an executor method

    def load(self):
        """The generated function ``run(ex, inputs, consts) -> list`` (``ex``: an ``Executor`` of this processor)."""
        scope = {"torch": torch, "aten": aten, "STEPS": self.steps, "Ref": Ref}
        exec(compile(self.source, f"<host program {self.name}>", "exec"), scope)
        return scope["run"]


def generate(scheduled, plan: Plan | None = None) -> dict[str, HostProgram]:
    """``{processor: HostProgram}`` for the plan of ``scheduled`` (or ``plan``)."""
    plan = plan or scheduled.plan
    out = {}
    for pname, prog in lower(scheduled, plan).items():
        lines = ["def run(ex, inputs, consts):",
                 "    env = {}",
                 "    def val(a):",
                 "        if isinstance(a, Ref):",
                 "            return env.get(a.name)",
                 "        if isinstance(a, (list, tuple)):",
                 "            return type(a)(val(x) for x in a)",
                 "        return a",
                 "    def take(name):                     # this processor's part of an input",
                 "        t = inputs[name]",
                 "        return ex._here(ex.shard(t, ex.plan.input_specs[name])) if isinstance(t, torch.Tensor) else t"]
        for name in plan.inputs:
            lines.append(f"    {name} = take({name!r})")
        hp = HostProgram(pname, prog.rank, "", plan.steps)
        defined = set(plan.inputs)
        for i, st in prog.steps:
            for r in _names(st):
                if r not in defined:                  # a value that does not exist on this processor
                    lines.append(f"    {r} = None")
                    defined.add(r)
            direct = _direct(st, plan.mesh.coords(prog.rank)) if st.op == "call" else None
            if st.op == "const":
                text = f"ex._here(consts({st.target!r}))"
            elif st.op == "alias":
                text = st.args[0].name
            elif st.op == "collective":           # (a bucketed reduction goes out on its own here: same sums)
                text = f"ex.collective(STEPS[{i}], {st.args[0].name})"
                hp.through_executor += 1
            elif direct is not None:
                text = direct
                hp.direct += 1
            else:
                # whatever the executor treats specially runs through it, on the values computed so far
                refs = sorted(set(_names(st)))
                lines.append(f"    env.update({{{', '.join(f'{r!r}: {r}' for r in refs)}}})")
                text = f"ex.run_step(STEPS[{i}], env, val)"
                hp.through_executor += 1
            lines.append(f"    {st.out} = {text}")
            defined.add(st.out)
        rets = []
        for o in plan.outputs:
            rets.append(repr(o[1]) if isinstance(o, tuple) else (o if o in defined else "None"))
        lines.append(f"    return [{', '.join(rets)}]")
        hp.source = "\n".join(lines) + "\n"
        out[pname] = hp
    return out


def _names(st) -> list[str]:
    found: list[str] = []

    def walk(o):
        if isinstance(o, Ref):
            found.append(o.name)
        elif isinstance(o, (list, tuple)):
            for x in o:
                walk(x)
        elif isinstance(o, dict):
            for x in o.values():
                walk(x)
    walk(st.args)
    walk(st.kwargs)
    return found
