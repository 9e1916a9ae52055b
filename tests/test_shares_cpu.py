"""Share solver, allocator and helpers."""
import math

import torch

from mesh_b200.compiler import Program, compile_module, shares
from mesh_b200.models.llama import Decoder, megatron
from mesh_b200.runtime.allocate import Allocator, equal_finish, separators, shift


def test_equal_finish_and_allocator_converges():
    ints, real, T = equal_finish(4096, 64, [64, 64], [math.inf, math.inf], [0.0, 0.0], [1.0, 3.0])
    assert sum(ints) == 4096 and abs(real[0] / real[1] - 3.0) < 1e-9 and ints[0] % 64 == 0
    # rank 1 is 4x slower than rank 0; the allocator finds ~4:1 from observed times alone
    speed = [1.0, 0.25]
    alloc = Allocator([2048, 2048], 64, [64, 64], [(0, 1e-3, 1.0, 1e-4)] * 2, [1e-6, 1e-6], forget=0.9, step=1.0)
    s = [2048, 2048]
    for _ in range(12):
        s = alloc([s[i] / speed[i] * 1e-3 for i in range(2)])
    assert abs(s[0] / s[1] - 4.0) < 0.35 and sum(s) == 4096


def test_shift_and_separators():
    out = shift([10, 2, 2], [6, 6, 6], [lambda x: x] * 3)
    assert sum(out) == 14 and max(out) <= 6
    cuts = separators([0, 10, 20, 30, 40, 100, 110], [1, 1])
    assert cuts[0] == 0 and cuts[-1] == 6
    loads = [(110 - 0)]  # sanity: cut is monotone
    assert cuts == sorted(cuts)


def test_solved_shares_follow_supplied_rates():
    torch.manual_seed(0)
    m = Decoder(dim=64, heads=4, ffn=128, layers=1)
    x = torch.randn(2, 8, 64)
    procs = {"fast": (0, "cpu"), "slow": (0, "cpu")}
    sch = compile_module(m, (x,), procs, megatron(procs), loss=0)
    staged = shares.stages(sch, segment=lambda st: "model")
    costs = shares.supplied(staged, procs, {"fast": 3e9, "slow": 1e9})
    ratios = shares.solved(staged, costs, comm=0.0, upper=[1.0, 1.0])["model"]
    # replicated (unsharded) work costs the slow rank more, so the optimum leans a little past 3:1
    assert 2.9 < ratios[0] / ratios[1] < 3.6
    # the solved ratios are valid units for the placement
    sch2 = compile_module(m, (x,), procs, megatron(procs, units=ratios), loss=0)
    res = Program(sch2)(x)
    assert abs(float(res.outputs) - float(m(x))) < 1e-5
    assert shares.shifted((7, 1), (0.75, 0.75), lambda j, u: u[j]) == (6, 2)


def test_ragged_rows():
    r = shares.Ragged(torch.arange(12.0), torch.tensor([0, 2, 5, 9, 12]))
    (lengths, cuts), (values, vcuts) = shares.rows(r, [1, 1])
    assert lengths.tolist() == [2, 3, 4, 3] and cuts[0] == 0 and cuts[-1] == 4 and vcuts[-1] == 12


def test_coupled_share_solve_matches_a_reference_lp_solver():
    """The native simplex against scipy's HiGHS on random stage models (fixed costs, per-part coefficients, collective
    terms at the largest share, per-rank caps): same optimum, feasible shares."""
    import random
    import numpy as np
    from scipy.optimize import linprog
    from mesh_b200 import graph as G
    random.seed(0)
    bad = 0
    for trial in range(80):
        S, R, P = random.randint(1, 4), random.randint(1, 5), random.randint(1, 3)
        fixed = [[random.random() * 0.5 for _ in range(R)] for _ in range(S)]
        coef = [[[random.random() * 3 if random.random() < 0.7 else 0.0 for _ in range(P)] for _ in range(R)] for _ in range(S)]
        comm = [[random.random() * 0.3 for _ in range(P)] for _ in range(S)] if random.random() < 0.5 else None
        upper = [min(1.0, 1.0 / R + random.random() * 0.6) for _ in range(R)] if random.random() < 0.5 else None
        # LP: variables x[p][j] (P*R), t[s] (S), m[s][p] (S*P, max_j x[p][j] bound per stage... one m[p] suffices)
        nx = P * R; nt = S; nm = P
        c = np.zeros(nx + nt + nm); c[nx:nx + nt] = 1.0
        if comm is not None:
            for p in range(P): c[nx + nt + p] = sum(comm[s][p] for s in range(S))
        A, b = [], []
        for s in range(S):
            for j in range(R):
                row = np.zeros(nx + nt + nm)
                for p in range(P): row[p * R + j] = coef[s][j][p]
                row[nx + s] = -1.0
                A.append(row); b.append(-fixed[s][j])
        for p in range(P):
            for j in range(R):
                row = np.zeros(nx + nt + nm); row[p * R + j] = 1.0; row[nx + nt + p] = -1.0
                A.append(row); b.append(0.0)
        Aeq, beq = [], []
        for p in range(P):
            row = np.zeros(nx + nt + nm); row[p * R:(p + 1) * R] = 1.0
            Aeq.append(row); beq.append(1.0)
        bounds = [(0, upper[j] if upper else None) for p in range(P) for j in range(R)] + [(None, None)] * (nt + nm)
        ref = linprog(c, A_ub=np.array(A), b_ub=np.array(b), A_eq=np.array(Aeq), b_eq=np.array(beq), bounds=bounds, method="highs")
        try:
            x, obj = G.shares_coupled(fixed, coef, comm, upper)
            if ref.status != 0: bad += 1; print("ref infeasible but solved", trial)
            else:
                # evaluate our x under the true objective
                val = sum(max(fixed[s][j] + sum(coef[s][j][p] * x[p][j] for p in range(P)) for j in range(R)) + (sum(comm[s][p] * max(x[p]) for p in range(P)) if comm else 0.0) for s in range(S))
                feas = all(abs(sum(x[p]) - 1) < 1e-6 and min(x[p]) > -1e-9 and (upper is None or all(x[p][j] <= upper[j] + 1e-6 for j in range(R))) for p in range(P))
                if not feas or val > ref.fun + 1e-5 or abs(obj - val) > 1e-5:
                    bad += 1; print("subopt", trial, S, R, P, val, ref.fun, obj, feas)
        except ValueError as e:
            if ref.status == 0: bad += 1; print("we failed", trial, e, ref.fun)

    assert bad == 0
