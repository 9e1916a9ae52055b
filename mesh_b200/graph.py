"""Python access to the native graph library (csrc/graph/graph.cpp): levels, strided-view dependences,
lifetime colouring, coupled share solve, cycle mean, signature check.  Mirrors what rdma/mesh_graph.py wraps
of rdma/mesh-graph.c, restricted to what a uniform NVSwitch fabric still needs."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_double, c_int, c_int64

from . import _native


def _ia(xs):
    return (c_int * len(xs))(*[int(x) for x in xs])


def _la(xs):
    return (c_int64 * len(xs))(*[int(x) for x in xs])


def _da(xs):
    return (c_double * len(xs))(*[float(x) for x in xs])


def levels(n: int, edges: list[tuple[int, int]]) -> list[int]:
    """Longest-path level of every node; raises on a cycle."""
    out = (c_int * max(n, 1))()
    rc = _native.lib().mesh_graph_levels(c_int(n), c_int(len(edges)), _ia([e[0] for e in edges]), _ia([e[1] for e in edges]), out)
    if rc != 0:
        raise ValueError("graph has a cycle")
    return list(out)[:n]


def _view(base, sizes, strides, elem):
    sizes, strides = list(sizes), list(strides)
    return base, len(sizes), _la(sizes or [1]), _la(strides or [0]), elem


def views_overlap(a, b) -> bool:
    """``a``, ``b``: ``(base_bytes, sizes, strides_bytes, elem_bytes)``; exact for box-strided views."""
    ba, na, sa, ta, ea = _view(*a)
    bb, nb, sb, tb, eb = _view(*b)
    return bool(_native.lib().mesh_graph_views_overlap(c_int64(ba), c_int(na), sa, ta, c_int64(ea),
                                                      c_int64(bb), c_int(nb), sb, tb, c_int64(eb)))


def dependences(accesses: list[tuple]) -> list[tuple[int, int, str]]:
    """``accesses``: program-ordered ``(op, is_write, buffer, (base, sizes<=3, strides<=3, elem))``.
    Returns ``(earlier op, later op, "RAW" | "WAR" | "WAW")`` for every conflicting pair."""
    n = len(accesses)
    packed = []
    for _, _, _, (base, sizes, strides, elem) in accesses:
        sizes = list(sizes) + [1] * (3 - len(sizes))
        strides = list(strides) + [0] * (3 - len(strides))
        packed += [base, elem, *sizes, *strides]
    cap = max(16, n * n)
    es, ed, ek = (c_int * cap)(), (c_int * cap)(), (c_int * cap)()
    cnt = _native.lib().mesh_graph_dependences(c_int(n), _ia([a[0] for a in accesses]), _ia([int(a[1]) for a in accesses]),
                                               _ia([a[2] for a in accesses]), _la(packed), c_int(cap), es, ed, ek)
    kinds = ["RAW", "WAR", "WAW"]
    return [(es[i], ed[i], kinds[ek[i]]) for i in range(abs(cnt))]


def colour(lifetimes: list[tuple[int, int, int]], align: int = 256) -> tuple[list[int], int]:
    """``lifetimes``: ``(first step, last step, bytes)`` per buffer -> (byte offsets, total bytes)."""
    n = len(lifetimes)
    off = (c_int64 * max(n, 1))()
    L = _native.lib()
    L.mesh_graph_colour.restype = c_int64
    total = L.mesh_graph_colour(c_int(n), _ia([l[0] for l in lifetimes]), _ia([l[1] for l in lifetimes]),
                                _la([l[2] for l in lifetimes]), c_int64(align), off)
    return list(off)[:n], int(total)


def shares_coupled(fixed, coef, comm=None, upper=None):
    """Minimise ``sum_s [ max_j (fixed[s][j] + sum_p coef[s][j][p] * x[p][j]) + sum_p comm[s][p] * max_j x[p][j] ]``
    over shares ``x[p][j] >= 0``, ``sum_j x[p][j] = 1``, ``x[p][j] <= upper[j]``.  Returns ``(x[p][j], objective)``."""
    stages, ranks = len(fixed), len(fixed[0])
    parts = len(coef[0][0])
    flat_fixed = [fixed[s][j] for s in range(stages) for j in range(ranks)]
    flat_coef = [coef[s][j][p] for s in range(stages) for j in range(ranks) for p in range(parts)]
    flat_comm = [comm[s][p] for s in range(stages) for p in range(parts)] if comm is not None else [0.0] * (stages * parts)
    out = (c_double * (parts * ranks))()
    obj = c_double(0)
    rc = _native.lib().mesh_graph_shares_coupled(c_int(parts), c_int(ranks), c_int(stages), _da(flat_fixed), _da(flat_coef),
                                                 _da(flat_comm), _da(upper) if upper is not None else None, out,
                                                 ctypes.byref(obj))
    if rc != 0:
        raise ValueError("share solve: infeasible (caps sum below 1?)" if rc == 1 else "share solve: unbounded")
    return [[out[p * ranks + j] for j in range(ranks)] for p in range(parts)], obj.value


def cycle_mean(n: int, edges: list[tuple[int, int, float]]) -> float:
    L = _native.lib()
    L.mesh_graph_cycle_mean.restype = c_double
    return L.mesh_graph_cycle_mean(c_int(n), c_int(len(edges)), _ia([e[0] for e in edges]), _ia([e[1] for e in edges]),
                                   _da([e[2] for e in edges]))


def signature_check(sequences: list[list[int]]) -> int:
    """-1 when every member issues the same ordered operations, else the first differing position."""
    flat = [x for s in sequences for x in s]
    return _native.lib().mesh_graph_signature_check(c_int(len(sequences)), _ia([len(s) for s in sequences]), _la(flat or [0]))


# ------------------------------------------------------------------------------------------------ scheduling, routing
def longest_path(n: int, edges: list[tuple[int, int]], cost: list[float]) -> list[float]:
    """``tail[v]``: ``cost[v]`` plus the heaviest path after ``v``; ``max(tail)`` is the critical path."""
    out = (c_double * max(n, 1))()
    rc = _native.lib().mesh_graph_longest_path(c_int(n), c_int(len(edges)), _ia([e[0] for e in edges]), _ia([e[1] for e in edges]),
                                               _da(cost), out)
    if rc != 0:
        raise ValueError("graph has a cycle")
    return list(out)[:n]


def list_schedule(n: int, edges: list[tuple[int, int]], cost: list[float], procs: int):
    """Critical-path list scheduling on ``procs`` identical processors -> ``(start, processor, makespan)``."""
    start, proc, span = (c_double * max(n, 1))(), (c_int * max(n, 1))(), c_double(0)
    rc = _native.lib().mesh_graph_list_schedule(c_int(n), c_int(len(edges)), _ia([e[0] for e in edges]), _ia([e[1] for e in edges]),
                                                _da(cost), c_int(procs), start, proc, ctypes.byref(span))
    if rc != 0:
        raise ValueError("graph has a cycle" if rc == -1 else "need at least one processor")
    return list(start)[:n], list(proc)[:n], span.value


def chains(n: int, edges: list[tuple[int, int]]) -> tuple[list[int], int]:
    """Minimum chain cover of a DAG (Dilworth): ``(chain id per node, number of chains)``."""
    out = (c_int * max(n, 1))()
    k = _native.lib().mesh_graph_chains(c_int(n), c_int(len(edges)), _ia([e[0] for e in edges]), _ia([e[1] for e in edges]), out)
    if k < 0:
        raise ValueError("graph has a cycle")
    return list(out)[:n], k


def arborescence(n: int, edges: list[tuple[int, int, float]], root: int) -> tuple[list[int], float]:
    """Cheapest broadcast tree from ``root`` (Chu-Liu / Edmonds): ``(index of the edge entering each node, weight)``."""
    pe, total = (c_int * max(n, 1))(), c_double(0)
    rc = _native.lib().mesh_graph_arborescence(c_int(n), c_int(len(edges)), _ia([e[0] for e in edges]), _ia([e[1] for e in edges]),
                                               _da([e[2] for e in edges]), c_int(root), pe, ctypes.byref(total))
    if rc != 0:
        raise ValueError("some node cannot be reached from the root")
    return list(pe)[:n], total.value


def concurrent_flow(n: int, edges: list[tuple[int, int, float]], commodities: list[tuple[int, int, float]], eps: float = 0.05):
    """Largest fraction of every demand that fits at once (Garg-Koenemann) -> ``(lambda, flow[commodity][edge])``."""
    m, k = len(edges), len(commodities)
    flow = (c_double * max(1, m * k))()
    f = _native.lib().mesh_graph_concurrent_flow
    f.restype = c_double
    lam = f(c_int(n), c_int(m), _ia([e[0] for e in edges]), _ia([e[1] for e in edges]), _da([e[2] for e in edges]), c_int(k),
            _ia([c[0] for c in commodities]), _ia([c[1] for c in commodities]), _da([c[2] for c in commodities]), c_double(eps), flow)
    if lam < 0:
        raise ValueError("a commodity has no path")
    return lam, [list(flow[c * m:(c + 1) * m]) for c in range(k)]


def dot(n: int, edges: list[tuple[int, int]], labels: list[str] | None = None, groups: list[int] | None = None) -> str:
    """Graphviz text of a graph; ``groups[v]`` colours nodes by processor / chain."""
    palette = ["#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f"]
    lines = ["digraph mesh {", "  rankdir=LR;"]
    for v in range(n):
        attr = [f'label="{labels[v] if labels else v}"']
        if groups is not None:
            attr.append(f'style=filled fillcolor="{palette[groups[v] % len(palette)]}"')
        lines.append(f"  n{v} [{' '.join(attr)}];")
    lines += [f"  n{a} -> n{b};" for a, b in edges]
    lines.append("}")
    return "\n".join(lines) + "\n"
