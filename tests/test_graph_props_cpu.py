"""The native graph library against brute force on small random instances."""
import itertools
import random

from mesh_b200 import graph as G


def test_colouring_chains_paths_schedules_and_arborescences_on_random_graphs():
    random.seed(0)
    bad = 0
    # --- colouring: buffers alive at the same time never share bytes
    for t in range(60):
        n = random.randint(1, 12)
        lt = []
        for _ in range(n):
            s = random.randint(0, 10); lt.append((s, s + random.randint(0, 5), random.randint(1, 1000)))
        offs, total = G.colour(lt, align=64)
        for i in range(n):
            if offs[i] % 64 or offs[i] + lt[i][2] > total: bad += 1; print("colour bounds", lt, offs, total)
            for j in range(i):
                live = not (lt[i][1] < lt[j][0] or lt[j][1] < lt[i][0])
                share = not (offs[i] + lt[i][2] <= offs[j] or offs[j] + lt[j][2] <= offs[i])
                if live and share: bad += 1; print("colour clash", lt, offs)
    # --- chains: a valid cover, and as small as the largest antichain (brute force)
    for t in range(50):
        n = random.randint(1, 8)
        edges = [(i, j) for i in range(n) for j in range(i + 1, n) if random.random() < 0.3]
        reach = [[False] * n for _ in range(n)]
        for i, j in edges: reach[i][j] = True
        for k in range(n):
            for i in range(n):
                for j in range(n):
                    if reach[i][k] and reach[k][j]: reach[i][j] = True
        closure = [(i, j) for i in range(n) for j in range(n) if reach[i][j]]
        chain, k = G.chains(n, closure)
        groups = {}
        for v, c in enumerate(chain): groups.setdefault(c, []).append(v)
        for g in groups.values():
            for a, b in zip(g, g[1:]):
                if not reach[a][b]: bad += 1; print("not a chain", edges, chain)
        width = max(len(s) for r in range(1, n + 1) for s in itertools.combinations(range(n), r) if all(not reach[a][b] and not reach[b][a] for a, b in itertools.combinations(s, 2)))
        if k != width or len(groups) != k: bad += 1; print("width", edges, k, width)
    # --- longest path tails
    for t in range(50):
        n = random.randint(1, 9)
        edges = [(i, j) for i in range(n) for j in range(i + 1, n) if random.random() < 0.35]
        cost = [random.random() for _ in range(n)]
        tail = G.longest_path(n, edges, cost)
        ref = [0.0] * n
        for v in reversed(range(n)):
            ref[v] = cost[v] + max([ref[j] for i, j in edges if i == v], default=0.0)
        if max(abs(a - b) for a, b in zip(tail, ref)) > 1e-9: bad += 1; print("tail", edges)
        start, proc, span = G.list_schedule(n, edges, cost, 2)
        for i, j in edges:
            if start[j] + 1e-9 < start[i] + cost[i]: bad += 1; print("schedule order", edges)
        for a in range(n):
            for b in range(a):
                if proc[a] == proc[b] and not (start[a] + cost[a] <= start[b] + 1e-9 or start[b] + cost[b] <= start[a] + 1e-9): bad += 1; print("schedule overlap")
        if span + 1e-9 < max(ref) or span > sum(cost) + 1e-9: bad += 1; print("span", span, max(ref))
    # --- minimum arborescence vs brute force
    for t in range(50):
        n = random.randint(2, 5)
        edges = [(i, j, random.randint(1, 9) * 1.0) for i in range(n) for j in range(n) if i != j and random.random() < 0.6]
        best = None
        for choice in itertools.product(*[[e for e in edges if e[1] == v] or [None] for v in range(1, n)]):
            if any(c is None for c in choice): continue
            parent = {c[1]: c[0] for c in choice}
            ok = True
            for v in range(1, n):
                seen, u = set(), v
                while u != 0:
                    if u in seen: ok = False; break
                    seen.add(u); u = parent[u]
                if not ok: break
            if ok:
                cst = sum(c[2] for c in choice); best = cst if best is None else min(best, cst)
        try:
            par, cst = G.arborescence(n, edges, 0)
            if best is None: bad += 1; print("arb should fail", edges)
            elif abs(cst - best) > 1e-9: bad += 1; print("arb cost", edges, cst, best)
        except Exception:
            if best is not None: bad += 1; print("arb failed", edges, best)

    assert bad == 0


def test_strided_view_overlap_never_misses_a_shared_byte():
    random.seed(1)

    def elements(view):
        base, sizes, strides, elem = view
        out = set()
        for idx in itertools.product(*[range(s) for s in sizes]):
            first = base + sum(i * st for i, st in zip(idx, strides))
            out.update(range(first, first + elem))
        return out

    def view():
        elem = random.choice([1, 2, 4])
        nd = random.randint(1, 3)
        return (random.randint(0, 20) * elem, [random.randint(1, 4) for _ in range(nd)],
                [random.randint(1, 12) * elem for _ in range(nd)], elem)
    for _ in range(300):
        a, b = view(), view()
        if elements(a) & elements(b):
            assert G.views_overlap(a, b), (a, b)
