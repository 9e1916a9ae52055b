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
