"""``lower(scheduled)``: one straight-line program per processor.

The plan is SPMD: one list of steps that every processor walks, skipping what does not concern it.  Lowering makes that
explicit.  For each processor it works out which values exist there (a value placed on one processor exists only on
its owner; a call exists where all its operands do; a gather to an owner exists only at the owner ...), drops the
steps that produce nothing on that processor and are not collectives it must take part in, and prints the rest as a
Python function whose lines are the processor's calls and collectives, in order.  The text is what a person reads to
see what a processor will do (and what an archive can store next to the plan); running it goes through the same
executor as the interpreted plan, so both give the same numbers.  The reference lowers its scheduled programs the
same way, to one function per processor (compiler/mesh_compiler/lower.py; design/the-compiler.md:30-36).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .ir import Plan, Ref, Step
from .runtime import Executor


def _refs(obj, out):
    if isinstance(obj, Ref):
        out.append(obj.name)
    elif isinstance(obj, (tuple, list)):
        for o in obj:
            _refs(o, out)
    elif isinstance(obj, dict):
        for o in obj.values():
            _refs(o, out)


def _present_after(st: Step, here: dict[str, bool], coords: tuple, mesh) -> bool:
    """Does ``st`` leave a value on the processor at ``coords``?"""
    names: list[str] = []
    _refs(st.args, names)
    _refs(st.kwargs, names)
    have = all(here.get(n, True) for n in names)
    if st.op in ("const",):
        return True
    if st.op in ("call", "alias", "slice", "fused"):
        return have
    if st.op == "collective":
        m, verb = st.meta, st.target
        me = coords[m["axis"]]
        to, frm = m["to"], m["from"]
        if verb in ("reduce", "gather", "send_recv"):
            return getattr(to, "owner", None) == me
        if verb in ("broadcast", "scatter"):
            return True
        return have
    return have


def _takes_part(st: Step, here: dict[str, bool], coords: tuple) -> bool:
    """Collectives are joined by every processor of their axis that holds a piece, even if it keeps no result."""
    if st.op != "collective":
        return False
    names: list[str] = []
    _refs(st.args, names)
    m = st.meta
    if st.target in ("broadcast", "scatter"):
        return True
    return all(here.get(n, True) for n in names) or getattr(m["from"], "kind", "") == "O"


@dataclass
class ProcessorProgram:
    name: str
    rank: int
    steps: list = field(default_factory=list)          # (index in the plan, step)
    source: str = ""

    def run(self, plan: Plan, inputs: dict, consts, coll, device=torch.device("cpu")) -> list:
        """Execute this processor's steps (``coll``: the collectives object of the executor family)."""
        ex = Executor(plan, self.rank, coll, device)
        keep = {i for i, _ in self.steps}
        sub = Plan(plan.mesh, [st for i, st in enumerate(plan.steps) if i in keep], plan.inputs, plan.input_specs,
                   plan.outputs, plan.output_specs, plan.transfers, plan.full_shapes, plan.dtypes)
        ex.plan = sub
        # values that do not exist here read as None, which is how the executor marks "lives elsewhere"
        class _Env(dict):
            def __missing__(self, k):
                return None
        return _run_with_env(ex, inputs, consts, _Env())


def _run_with_env(ex: Executor, inputs: dict, consts, env) -> list:
    for name, full in inputs.items():
        env[name] = ex.shard(full, ex.plan.input_specs[name]) if isinstance(full, torch.Tensor) else full

    def val(a):
        if isinstance(a, Ref):
            return env[a.name]
        if isinstance(a, (list, tuple)):
            return type(a)(val(x) for x in a)
        return a
    from .placement import local_indices
    for st in ex.plan.steps:
        if st.op == "const":
            env[st.out] = consts(st.target)
        elif st.op == "alias":
            env[st.out] = env[st.args[0].name]
        elif st.op == "slice":
            src = env[st.args[0].name]
            s, ax = st.meta["to"], st.meta["axis"]
            env[st.out] = None if src is None else ex._index(src, s.dim, local_indices(s, ex.coords[ax], src.shape[s.dim]))
        elif st.op == "collective":
            env[st.out] = ex.collective(st, env[st.args[0].name])
        elif st.op == "fused" and st.target == "rms_norm":
            env[st.out] = ex.rms_norm(st, env[st.args[0].name], env[st.args[1].name] if len(st.args) > 1 else None)
        elif st.op == "fused":
            env[st.out] = ex.fused(st, env[st.args[0].name], env[st.args[1].name], env)
        else:
            env[st.out] = ex.call(st, val)
    return [o[1] if isinstance(o, tuple) else env[o] for o in ex.plan.outputs]


def _fmt(a) -> str:
    if isinstance(a, Ref):
        return a.name
    if isinstance(a, (list, tuple)):
        inner = ", ".join(_fmt(x) for x in a)
        return f"[{inner}]" if isinstance(a, list) else f"({inner}{',' if len(a) == 1 else ''})"
    if isinstance(a, torch.dtype) or isinstance(a, torch.device):
        return str(a)
    return repr(a)


def _line(st: Step) -> str:
    if st.op == "const":
        return f"{st.out} = constant({st.target!r})"
    if st.op == "alias":
        return f"{st.out} = {_fmt(st.args[0])}"
    if st.op == "slice":
        return f"{st.out} = local_slice({_fmt(st.args[0])}, axis={st.meta['axis']}, to={st.meta['to']!r})"
    if st.op == "collective":
        m = st.meta
        extra = f", left={m['left']}, right={m['right']}" if st.target in ("halo", "halo_back") else ""
        return f"{st.out} = {st.target}({_fmt(st.args[0])}, axis={m['axis']}, channel={m.get('channel')}{extra})   # {m['from']!r} -> {m['to']!r}"
    if st.op == "fused" and st.target == "rms_norm":
        return f"{st.out} = rms_norm({', '.join(_fmt(a) for a in st.args)}, eps={st.meta['eps']})"
    if st.op == "fused":
        return f"{st.out} = fused_{st.target}({', '.join(_fmt(a) for a in st.args)}, axis={st.meta['axis']}, channel={st.meta.get('channel')})"
    name = getattr(st.target, "__name__", None) or str(st.target)
    pkg = str(st.target).replace("aten.", "") if str(st.target).startswith("aten.") else name
    args = ", ".join([_fmt(a) for a in st.args] + [f"{k}={_fmt(v)}" for k, v in st.kwargs.items()])
    return f"{st.out} = {pkg}({args})"


def lower(scheduled, plan: Plan | None = None) -> dict[str, ProcessorProgram]:
    """``{processor name: ProcessorProgram}`` for the plan of ``scheduled`` (or for ``plan``, e.g. a fused one)."""
    plan = plan or scheduled.plan
    mesh = plan.mesh
    out = {}
    for rank, pname in enumerate(mesh.names):
        coords = mesh.coords(rank)
        here: dict[str, bool] = {}
        for name in plan.inputs:
            specs = plan.input_specs.get(name, ())
            here[name] = all(not (s.kind == "O" and s.owner != coords[a]) for a, s in enumerate(specs))
        prog = ProcessorProgram(pname, rank)
        lines = [f"def processor_{pname}({', '.join(n for n in plan.inputs if here[n])}):"]
        for i, st in enumerate(plan.steps):
            present = _present_after(st, here, coords, mesh)
            here[st.out] = present
            if present or _takes_part(st, here, coords):
                prog.steps.append((i, st))
                text = _line(st)
                if not present:
                    text = text.split(" = ", 1)[1] + "   # takes part, keeps nothing"
                lines.append("    " + text)
        rets = [(_fmt(Ref(o)) if here.get(o, True) else "None") if isinstance(o, str) else repr(o[1]) for o in plan.outputs]
        lines.append(f"    return [{', '.join(rets)}]")
        prog.source = "\n".join(lines) + "\n"
        out[pname] = prog
    return out
