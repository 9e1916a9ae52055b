"""Analysis of a program made of calls: which calls depend on which, how many can be outstanding, which commute.

The reference analyses a captured *program of calls* before planning it (compiler/mesh_compiler/schedule.py:420-1010):
a dependence relation between the calls (Bernstein's conditions over the storages they read and write), a cover of the
calls by the fewest chains (Dilworth), from which the number of executions of one function that can be in flight
follows, and a symbolic test of whether two successive calls of a function through one of its inputs give the same
result in either order (Rinard and Diniz's commutativity analysis), which turns a chain of accumulating calls into a
reduction that may be reordered.

Here the capture inlines the calls into one graph in which every node remembers the submodule call it came from
(``torch.export`` keeps the module stack), so

* :func:`analyse` recovers the call instances, the flow of values between them (a value that passes through glue
  outside any function carries its producers along), the transitive closure, the chain cover and per-function widths
  and the critical path (node counts as costs) through ``mesh_b200.graph``;
* :func:`commutes` interprets an exported function body over symbols.  Values are polynomials over atoms with exact
  rational coefficients - sums and products are put in one normal form by construction, anything else is an opaque atom
  keyed by its operator and normalised operands - so two compositions are equal exactly when their polynomials are.
"""
from __future__ import annotations

import dataclasses
from fractions import Fraction

import torch

from .. import graph as G
from .ir import Exported

aten = torch.ops.aten


# ----------------------------------------------------------------------------- symbolic values
class Poly:
    """A polynomial: ``{monomial: coefficient}`` with a monomial a sorted tuple of hashable atoms."""

    __slots__ = ("terms",)

    def __init__(self, terms: dict | None = None):
        self.terms = {m: c for m, c in (terms or {}).items() if c != 0}

    @staticmethod
    def atom(key) -> "Poly":
        return Poly({(key,): Fraction(1)})

    @staticmethod
    def const(value) -> "Poly":
        return Poly({(): Fraction(value).limit_denominator(1 << 30) if isinstance(value, float) else Fraction(value)})

    def key(self):
        return tuple(sorted(((m, c) for m, c in self.terms.items()), key=repr))

    def __eq__(self, other):
        return isinstance(other, Poly) and self.terms == other.terms

    def __hash__(self):
        return hash(self.key())

    def __add__(self, other):
        out = dict(self.terms)
        for m, c in other.terms.items():
            out[m] = out.get(m, 0) + c
        return Poly(out)

    def __neg__(self):
        return Poly({m: -c for m, c in self.terms.items()})

    def __sub__(self, other):
        return self + (-other)

    def __mul__(self, other):
        out: dict = {}
        for ma, ca in self.terms.items():
            for mb, cb in other.terms.items():
                m = tuple(sorted(ma + mb, key=repr))
                out[m] = out.get(m, 0) + ca * cb
        return Poly(out)

    def __repr__(self):
        return "Poly(" + " + ".join(f"{c}*{'*'.join(map(str, m)) or '1'}" for m, c in self.terms.items()) + ")"


def _lift(x):
    if isinstance(x, Poly):
        return x
    if isinstance(x, bool):
        return Poly.const(int(x))
    if isinstance(x, (int, float)):
        return Poly.const(x)
    return None


def _frozen(x):
    if isinstance(x, Poly):
        return ("poly", x.key())
    if isinstance(x, (list, tuple)):
        return tuple(_frozen(v) for v in x)
    if isinstance(x, dict):
        return tuple(sorted((k, _frozen(v)) for k, v in x.items()))
    if isinstance(x, (torch.dtype, torch.device, torch.layout, torch.memory_format)):
        return str(x)
    return x


_RING = {aten.add.Tensor: "add", aten.add.Scalar: "add", aten.sub.Tensor: "sub", aten.sub.Scalar: "sub",
         aten.mul.Tensor: "mul", aten.mul.Scalar: "mul", aten.neg.default: "neg", aten.rsub.Scalar: "rsub",
         aten.div.Tensor: "div", aten.div.Scalar: "div"}
_IDENTITY = {aten.clone.default, aten.alias.default, aten.detach.default, aten.contiguous.default
             if hasattr(aten, "contiguous") else aten.clone.default, aten.lift_fresh_copy.default}


class Symbolic(torch.fx.Interpreter):
    """Runs a graph over :class:`Poly` values."""

    def call_function(self, target, args, kwargs):
        kind = _RING.get(target)
        if kind is not None:
            a = _lift(args[0])
            b = _lift(args[1]) if len(args) > 1 else None
            scale = _lift(kwargs.get("alpha", 1))
            if a is not None and (kind == "neg" or b is not None):
                if kind == "neg":
                    return -a
                if kind == "mul":
                    return a * b
                if kind == "div":
                    if set(b.terms) == {()}:                          # division by a constant is a scaling
                        return a * Poly({(): 1 / b.terms[()]})
                    return Poly.atom((str(target), _frozen(args), _frozen(kwargs)))
                if kind == "add":
                    return a + scale * b
                if kind == "sub":
                    return a - scale * b
                return b - scale * a                                 # rsub: other - alpha * self
        if target in _IDENTITY and isinstance(args[0], Poly):
            return args[0]
        import operator
        if target is operator.getitem and isinstance(args[0], (tuple, list)):
            return args[0][args[1]]
        return Poly.atom((str(target), _frozen(args), _frozen(kwargs)))


def commutes(function: Exported, k: int) -> bool:
    """Do two successive calls of ``function``, the first's result passed as the second's user input ``k``, give the
    same final result whichever of the two calls runs first?  (Each call has its own other inputs; state is shared.)"""
    gm = function.graph_module
    names = [n.name for n in gm.graph.nodes if n.op == "placeholder"]
    users = list(function.user_inputs)
    if not 0 <= k < len(users):
        raise IndexError(f"function has {len(users)} user inputs")
    through = users[k]
    result = next(i for i, (kind, _) in enumerate(function.outputs) if kind == "user")

    def run(receiver: Poly, call: int) -> Poly:
        args = []
        for name in names:
            if name == through:
                args.append(receiver)
            elif name in users:
                args.append(Poly.atom(("input", call, name)))
            else:
                args.append(Poly.atom(("state", name)))
        out = Symbolic(gm).run(*args, enable_io_processing=False)
        out = out[result] if isinstance(out, (tuple, list)) else out
        return out if isinstance(out, Poly) else Poly.atom(("value", _frozen(out)))

    start = Poly.atom(("receiver",))
    return run(run(start, 1), 2) == run(run(start, 2), 1)


# ----------------------------------------------------------------------------- the calls of a captured program
@dataclasses.dataclass
class CallAnalysis:
    calls: list            # (function, call-site key) in first-appearance order
    nodes: list            # how many graph nodes each call has
    edges: list            # (producer call, consumer call): a value flows
    closure: list          # per call: the set of calls it transitively depends on
    chains: list           # chain id per call of a fewest-chains cover of the dependence order
    width: int             # number of chains = the most calls that are pairwise independent
    widths: dict           # per function: the same, among its own calls
    critical: list         # the calls on a longest dependence path (node counts as costs)
    glue: int              # graph nodes outside every named function
    commuting: dict        # function -> {input position: True | False}, where bodies were supplied

    def outstanding(self, function: str) -> int:
        """How many executions of ``function`` can be in flight at once."""
        return self.widths.get(function, 0)

    def summary(self) -> dict:
        seen: dict = {}
        label = []
        for f, _ in self.calls:                                      # a#0, a#1, ...: the calls of one function in order
            label.append(f"{f}#{seen.get(f, 0)}")
            seen[f] = seen.get(f, 0) + 1
        return {"calls": len(self.calls), "edges": len(self.edges), "width": self.width, "widths": dict(self.widths),
                "critical_path": [label[i] for i in self.critical], "glue_nodes": self.glue,
                "commuting": {f: dict(v) for f, v in self.commuting.items()}}


def _instance(node, names: set):
    """The innermost named function whose call ``node`` was traced in: ``(function, call-site key)`` or None."""
    stack = node.meta.get("nn_module_stack") or {}
    found = None
    for key, (qual, _cls) in stack.items():
        if qual in names:
            found = (qual, key)
    return found


def analyse(exported: Exported, functions, bodies: dict | None = None) -> CallAnalysis:
    """``functions``: submodule qualified names (or callables with ``__name__``); ``bodies``: optionally each function's
    own :class:`Exported` (from exporting the submodule alone), for the commutativity test of its chains."""
    names = {f if isinstance(f, str) else getattr(f, "__name__", str(f)) for f in functions}
    index: dict = {}
    calls, counts = [], []
    origin: dict[str, frozenset] = {}
    edges: set = set()
    glue = 0
    for node in exported.graph_module.graph.nodes:
        if node.op == "placeholder":
            origin[node.name] = frozenset()
            continue
        if node.op == "output":
            continue
        sources = frozenset().union(*[origin.get(a.name, frozenset()) for a in node.all_input_nodes]) if node.all_input_nodes else frozenset()
        inst = _instance(node, names) if node.op == "call_function" else None
        if inst is None:
            glue += node.op == "call_function"
            origin[node.name] = sources                           # glue passes its producers on
            continue
        if inst not in index:
            index[inst] = len(calls)
            calls.append(inst)
            counts.append(0)
        me = index[inst]
        counts[me] += 1
        for s in sources:
            if s != me:
                edges.add((s, me))
        origin[node.name] = frozenset([me])
    n = len(calls)
    edge_list = sorted(edges)
    closure = [set() for _ in range(n)]
    preds = [[] for _ in range(n)]
    for a, b in edge_list:
        preds[b].append(a)
    for b in range(n):                                            # first-appearance order is a topological order
        for a in preds[b]:
            closure[b] |= closure[a] | {a}
    full = [(a, b) for b in range(n) for a in sorted(closure[b])]
    chain_of, width = G.chains(n, full) if n else ([], 0)
    widths = {}
    for f in sorted(names):
        mine = [i for i, (q, _) in enumerate(calls) if q == f]
        local = {c: j for j, c in enumerate(mine)}
        sub = [(local[a], local[b]) for b in mine for a in closure[b] if a in local]
        widths[f] = G.chains(len(mine), sub)[1] if mine else 0
    critical = []
    if n:
        tail = G.longest_path(n, edge_list, [float(c) for c in counts])     # cost of the call plus the heaviest path after it
        succs = [[] for _ in range(n)]
        for a, b in edge_list:
            succs[a].append(b)
        at = max(range(n), key=lambda i: tail[i])
        while True:
            critical.append(at)
            if not succs[at]:
                break
            at = max(succs[at], key=lambda i: tail[i])
    commuting: dict = {}
    for f, body in (bodies or {}).items():
        commuting[f] = {k: commutes(body, k) for k in range(len(body.user_inputs))}
    return CallAnalysis(calls, counts, edge_list, closure, list(chain_of), int(width), widths, critical, int(glue), commuting)
