"""Native graph library: levels, strided-view overlap, dependences, colouring, share solve (vs scipy), signature."""
import itertools
import random

import pytest

from mesh_b200 import graph


def test_levels_and_cycle():
    assert graph.levels(5, [(0, 1), (1, 2), (0, 2), (3, 4)]) == [0, 1, 2, 0, 1]
    with pytest.raises(ValueError):
        graph.levels(2, [(0, 1), (1, 0)])


def _brute(a, b):
    def addrs(v):
        base, sizes, strides, elem = v
        out = set()
        for idx in itertools.product(*[range(s) for s in sizes]):
            o = base + sum(i * st for i, st in zip(idx, strides))
            out.update(range(o, o + elem))
        return out
    return bool(addrs(a) & addrs(b))


def test_views_overlap_matches_brute_force():
    rnd = random.Random(0)
    for _ in range(300):
        def view():
            nd = rnd.randint(1, 3)
            return (rnd.randint(0, 40), [rnd.randint(1, 4) for _ in range(nd)], [rnd.choice([2, 4, 8, 16, 24, 32]) for _ in range(nd)], rnd.choice([2, 4]))
        a, b = view(), view()
        assert graph.views_overlap(a, b) == _brute(a, b), (a, b)
    # columns of a row-major matrix: even and odd columns never meet
    assert not graph.views_overlap((0, [8, 4], [64, 16], 8), (8, [8, 4], [64, 16], 8))


def test_dependences_kinds():
    v = lambda base, n: (base, [n], [4], 4)
    acc = [(0, True, 0, v(0, 8)), (1, False, 0, v(16, 4)), (2, True, 0, v(0, 4)), (3, False, 1, v(0, 8)), (4, True, 0, v(16, 2))]
    deps = set(graph.dependences(acc))
    assert (0, 1, "RAW") in deps and (0, 2, "WAW") in deps and (1, 4, "WAR") in deps
    assert not any(3 in (a, b) for a, b, _ in deps)


def test_colour_no_overlap_of_live_buffers():
    rnd = random.Random(1)
    life = []
    for _ in range(40):
        s = rnd.randint(0, 30)
        life.append((s, s + rnd.randint(0, 10), rnd.randint(1, 1000)))
    off, total = graph.colour(life, align=64)
    for i, j in itertools.combinations(range(len(life)), 2):
        if not (life[i][1] < life[j][0] or life[j][1] < life[i][0]):
            assert off[i] + life[i][2] <= off[j] or off[j] + life[j][2] <= off[i]
    assert total <= sum(((l[2] + 63) // 64) * 64 for l in life)
    assert total < 0.7 * sum(l[2] for l in life)          # reuse actually happens


def test_shares_coupled_against_scipy():
    from scipy.optimize import linprog
    import numpy as np
    rnd = random.Random(2)
    for trial in range(12):
        parts, ranks, stages = rnd.randint(1, 3), rnd.randint(2, 4), rnd.randint(1, 5)
        fixed = [[rnd.random() * 0.2 for _ in range(ranks)] for _ in range(stages)]
        coef = [[[rnd.random() * (1 + 3 * j) for _ in range(parts)] for j in range(ranks)] for _ in range(stages)]
        comm = [[rnd.random() * 0.3 for _ in range(parts)] for _ in range(stages)]
        upper = [0.9] * ranks
        x, obj = graph.shares_coupled(fixed, coef, comm, upper)
        nx = parts * ranks
        n = nx + stages + parts
        c = np.zeros(n); c[nx:nx + stages] = 1
        for p in range(parts):
            c[nx + stages + p] = sum(comm[s][p] for s in range(stages))
        A, b = [], []
        for s in range(stages):
            for j in range(ranks):
                row = np.zeros(n)
                for p in range(parts):
                    row[p * ranks + j] = coef[s][j][p]
                row[nx + s] = -1
                A.append(row); b.append(-fixed[s][j])
        for p in range(parts):
            for j in range(ranks):
                row = np.zeros(n); row[p * ranks + j] = 1; row[nx + stages + p] = -1
                A.append(row); b.append(0)
        Aeq = np.zeros((parts, n)); beq = np.ones(parts)
        for p in range(parts):
            Aeq[p, p * ranks:(p + 1) * ranks] = 1
        bounds = [(0, 0.9)] * nx + [(None, None)] * stages + [(0, None)] * parts
        ref = linprog(c, A_ub=np.array(A), b_ub=np.array(b), A_eq=Aeq, b_eq=beq, bounds=bounds)
        assert ref.status == 0
        assert abs(obj - ref.fun) < 1e-6 * max(1, abs(ref.fun)), (trial, obj, ref.fun)
        for p in range(parts):
            assert abs(sum(x[p]) - 1) < 1e-8 and max(x[p]) <= 0.9 + 1e-9


def test_cycle_mean_and_signature():
    assert abs(graph.cycle_mean(3, [(0, 1, 1.0), (1, 2, 2.0), (2, 0, 3.0)]) - 2.0) < 1e-12
    assert graph.cycle_mean(2, [(0, 1, 1.0)]) == -1.0
    assert graph.signature_check([[1, 2, 3], [1, 2, 3]]) == -1
    assert graph.signature_check([[1, 2, 3], [1, 9, 3]]) == 1
    assert graph.signature_check([[1, 2], [1, 2, 3]]) == 2


def test_longest_path_list_schedule_and_chains():
    from mesh_b200 import graph as G
    # diamond with a tail: 0 -> {1, 2} -> 3 -> 4
    edges = [(0, 1), (0, 2), (1, 3), (2, 3), (3, 4)]
    cost = [1.0, 5.0, 2.0, 1.0, 1.0]
    tail = G.longest_path(5, edges, cost)
    assert tail[0] == 8.0 and tail[2] == 4.0 and max(tail) == 8.0
    start, proc, span = G.list_schedule(5, edges, cost, procs=2)
    assert span == 8.0 and start[1] == 1.0 and start[2] == 1.0 and proc[1] != proc[2] and start[3] == 6.0
    _, _, span1 = G.list_schedule(5, edges, cost, procs=1)
    assert span1 == sum(cost)
    ids, k = G.chains(5, edges)
    assert k == 2 and ids[1] != ids[2]                     # the only antichain of size 2 is {1, 2}
    # an antichain of 4 independent nodes needs 4 chains
    assert G.chains(4, [])[1] == 4
    txt = G.dot(5, edges, groups=ids)
    assert txt.startswith("digraph") and "n0 -> n1" in txt


def test_arborescence_and_concurrent_flow():
    from mesh_b200 import graph as G
    # classic Edmonds example with a cycle 1 -> 2 -> 3 -> 1 that must be broken
    edges = [(0, 1, 10.0), (0, 2, 12.0), (0, 3, 9.0), (1, 2, 2.0), (2, 3, 3.0), (3, 1, 1.0)]
    pe, total = G.arborescence(4, edges, 0)
    assert pe[0] == -1 and abs(total - 12.0) < 1e-9          # 0->3 (9), 3->1 (1), 1->2 (2)
    assert {edges[e][:2] for e in pe[1:]} == {(0, 3), (3, 1), (1, 2)}
    # two commodities sharing one link of capacity 10: each wants 10 -> half of each fits
    fedges = [(0, 2, 100.0), (1, 2, 100.0), (2, 3, 10.0), (3, 4, 100.0), (3, 5, 100.0)]
    lam, flow = G.concurrent_flow(6, fedges, [(0, 4, 10.0), (1, 5, 10.0)], eps=0.05)
    assert 0.42 < lam <= 0.5 + 1e-9
    assert abs(flow[0][2] - lam * 10) < 1e-6 and flow[0][2] + flow[1][2] <= 10 + 1e-6
    # a parallel path doubles it
    lam2, _ = G.concurrent_flow(6, fedges + [(2, 3, 10.0)], [(0, 4, 10.0), (1, 5, 10.0)], eps=0.05)
    assert lam2 > 0.85
