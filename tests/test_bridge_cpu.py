"""Declared transfers, lifetimes and workspace layout of a plan; a prepared program with several input sets."""
import pytest
import torch

from mesh_b200.compiler import compile_module, prepare, workspace
from mesh_b200.compiler import schedule as S
from mesh_b200.models.llama import Block, megatron
from mesh_b200.runtime.rendezvous import MeshStale


def _compiled():
    torch.manual_seed(0)
    m = torch.nn.Sequential(Block(64, 4, 128)).eval()
    x = torch.randn(2, 16, 64)
    procs = {"a": (0, "cpu"), "b": (0, "cpu")}
    return m, x, compile_module(m, (x,), procs, megatron(procs))


def test_declared_transfers_carry_their_events_in_step_order():
    _, _, sch = _compiled()
    ds = S.declarations(sch.plan)
    assert len(ds) == 2 and all(d.verb == "all_reduce" for d in ds)          # the two all-reduces of a Megatron block
    for d in ds:
        assert d.produced < d.at < d.read <= d.consumed
        assert sch.plan.steps[d.at].out == d.result and d.nbytes > 0
    assert S.horizon(sch.plan, 3) == 3
    edges = S.carried(sch.plan, copies=2)
    assert any(e[2] == 2 and e[1].startswith("write:") for e in edges)        # inputs: write after read, lag = copies
    assert sum(1 for e in edges if e[2] == 1) == len(ds)                      # collectives: lag 1


def test_workspace_shares_bytes_between_values_that_do_not_overlap():
    _, _, sch = _compiled()
    w = workspace(sch, copies=2)
    assert 0 < w["bytes_per_copy"] < w["bytes_unshared"]
    lt = {name: (a, b, n) for name, a, b, n in S.lifetimes(sch.plan)}
    names = list(w["offsets"])
    # no two values that are alive at the same step overlap in a copy; the copies are disjoint
    for i, p in enumerate(names):
        for q in names[i + 1:]:
            (a0, a1, an), (b0, b1, bn) = lt[p], lt[q]
            if a0 <= b1 and b0 <= a1 and an and bn:
                po, qo = w["offsets"][p][0], w["offsets"][q][0]
                assert po + an <= qo or qo + bn <= po, (p, q)
    assert all(o[1] >= w["bytes_per_copy"] for o in w["offsets"].values())


def test_prepared_program_rotates_input_sets_and_refuses_a_stale_view():
    m, x, sch = _compiled()
    pr = prepare(sch, (x,), copies=2)
    outs = []
    for step in range(4):
        ins = pr.inputs()
        ins[0].copy_(x * (step + 1))
        b = pr.start()
        assert b == step and pr.ended(b)
        outs.append(pr.result(b))
    for step, o in enumerate(outs):
        assert torch.allclose(o, m(x * (step + 1)), atol=1e-5)
    with pytest.raises(KeyError):
        pr.result(0)                                         # held for `copies` executions only

    class _Rdv:                                              # a membership view that moves
        epoch = 0

        def check_epoch(self, e):
            if e != self.epoch:
                raise MeshStale("view moved")
    rdv = _Rdv()
    pr2 = prepare(sch, (x,), copies=1, rdv=rdv)
    pr2.start()
    rdv.epoch = 1
    with pytest.raises(MeshStale):
        pr2.start()


def test_workspace_carries_the_planned_transfers():
    """The prepared program's plan information includes the native planner's view of its transfers: the gradient
    reductions of a data-parallel step travel as few demands (buckets), every transfer has an algorithm, a place in the
    order of its axis and the time its reader waits; a small bucket size gives more demands."""
    import torch

    from mesh_b200.compiler import compile_module
    from mesh_b200.compiler import schedule as S
    from mesh_b200.compiler.bridge import workspace
    from mesh_b200.models.llama import Decoder, data_parallel
    torch.manual_seed(1)
    m = Decoder(dim=32, heads=2, ffn=64, layers=2)
    x = torch.randn(4, 6, 32)
    procs = {f"p{i}": (0, "cpu") for i in range(2)}
    sch = compile_module(m, (x,), procs, data_parallel(procs), loss=0)
    ws = workspace(sch)
    planned = ws["planned"]
    n = len(sch.plan.transfers)
    assert len(planned["transfers"]) == n and planned["summary"]["demands"] < n
    assert all(t["algo"] in ("one_shot", "two_shot", "nvls", "copy_engine") and t["pieces"] >= 1 for t in planned["transfers"])
    small = S.planned(sch.plan, bucket_bytes=8 << 10)
    assert small["summary"]["demands"] > planned["summary"]["demands"]
    assert abs(small["summary"]["exposed_us"] - sum({t["demand"]: t["exposed_us"] for t in small["transfers"]}.values())) < 1e-6


def test_workspace_states_the_steady_state_of_repeated_starts():
    """``workspace()["pipeline"]``: period, latency and copies from the native modulo scheduler over the plan's steps;
    ``prepare(copies=None)`` takes that many sets of buffers."""
    import torch
    from mesh_b200.compiler import compile_module, prepare, workspace
    from mesh_b200.models.llama import Decoder, megatron
    torch.manual_seed(0)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1).eval()
    x = torch.randn(2, 8, 32)
    procs = {f"p{i}": (0, "cpu") for i in range(2)}
    sch = compile_module(m, (x,), procs, megatron(procs))
    pipe = workspace(sch, 2)["pipeline"]
    assert pipe["period_us"] >= pipe["resource_bound_us"] > 0 and pipe["latency_us"] > 0
    assert pipe["copies"] == max(1, -(-int(pipe["latency_us"] / pipe["period_us"] * 1e6) // 10 ** 6))
    assert pipe["bound_by"] in ("compute", "dependences") or pipe["bound_by"].startswith("links of axis")
    # transfers that cost more than the compute between them: the links set the period and executions overlap
    from mesh_b200.compiler import schedule
    slow = schedule.pipelined(sch.plan, step_us=0.01)
    assert slow["bound_by"].startswith("links") and slow["copies"] >= 1
    p = prepare(sch, (x,), copies=None)
    assert p.copies == min(4, max(1, pipe["copies"]))
    p.start(x)
    assert torch.allclose(p.result(), m(x), atol=1e-5)


def test_steady_state_from_observed_step_times():
    """Measured step times (``observe``) in place of the modelled ones: the period is at least the measured compute."""
    import torch
    from mesh_b200.compiler import Program, compile_module, schedule
    from mesh_b200.compiler.observe import observe
    from mesh_b200.models.llama import Decoder, megatron
    torch.manual_seed(0)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1).eval()
    x = torch.randn(2, 8, 32)
    procs = {f"p{i}": (0, "cpu") for i in range(2)}
    prog = Program(compile_module(m, (x,), procs, megatron(procs)))
    report = observe(prog, x)
    pipe = schedule.pipelined(prog.plan, observed=report)
    compute_us = sum(r["seconds"] for r in report["steps"] if r["op"] not in ("collective",)) * 1e6
    assert pipe["period_us"] >= 0.5 * compute_us and pipe["latency_us"] >= pipe["period_us"] * 0.5 and pipe["copies"] >= 1
