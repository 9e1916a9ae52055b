"""Static checkers: plan structure, and the counter protocols of the collective and exchange kernels."""
import torch

from mesh_b200.compiler.check import CommModel, Launch, check_plan, simulate


def test_compiled_plan_is_clean_and_damage_is_found():
    from mesh_b200.compiler.driver import compile_module
    from mesh_b200.models.llama import Decoder, megatron
    torch.manual_seed(0)
    m = Decoder(dim=64, heads=4, ffn=128, layers=1)
    procs = {"a": (0, "cpu"), "b": (0, "cpu")}
    sched = compile_module(m, (torch.randn(2, 8, 64),), procs, megatron(list(procs)))
    plan = next(iter(sched.plans.values())) if hasattr(sched, "plans") else sched.plan
    assert check_plan(plan) == []
    # damage: use before definition, double definition, bad axis
    import copy
    bad = copy.deepcopy(plan)
    bad.steps[0], bad.steps[-1] = bad.steps[-1], bad.steps[0]
    assert any("before it is defined" in p for p in check_plan(bad))
    bad = copy.deepcopy(plan)
    bad.steps.append(bad.steps[-1])
    assert any("second time" in p for p in check_plan(bad))
    bad = copy.deepcopy(plan)
    for st in bad.steps:
        if st.op == "collective":
            st.meta["axis"] = 7
            break
    assert any("axis 7" in p for p in check_plan(bad))


def _all(models):
    out = {}
    for m in models.values():
        out.update(m.programs())
    return out


def test_collective_sequences_complete_and_a_missing_rank_is_reported():
    W = 4
    models = {r: CommModel(r, W) for r in range(W)}
    for call in range(5):
        for r in range(W):
            if call == 4 and r == 2:
                continue
            models[r].collective(f"ar{call}", nblocks=8 if call % 2 else 148, two_step=call == 3)
    # rank 2 skipped the last collective: everyone else waits on it for ever
    stuck = simulate(_all(models))
    assert len(stuck) == 3 and all("ar4" in s for s in stuck)
    models[2].collective("ar4", nblocks=148)
    assert simulate(_all(models)) == []


def test_ring_exchange_of_messages_larger_than_the_ring():
    W, depth, piece = 4, 4, 1 << 20
    models = {r: CommModel(r, W, depth, piece) for r in range(W)}
    for r in range(W):
        models[r].exchange("ring", 64 << 20, dsts=[(r + 1) % W], src=(r - 1) % W, nb=3)    # 64 pieces, ring of 4
        models[r].collective("ar", nblocks=16)
        models[r].exchange("ring2", 3 << 20, dsts=[(r + 1) % W], src=(r - 1) % W)          # counter bases carry over
    assert simulate(_all(models)) == []


def test_send_before_recv_on_both_sides_deadlocks_only_beyond_the_ring():
    depth, piece = 4, 1 << 20
    for nbytes, should_hang in ((3 << 20, False), (4 << 20, False), (8 << 20, True)):
        models = {r: CommModel(r, 2, depth, piece) for r in range(2)}
        for r in range(2):
            # a send-only launch followed by a receive-only launch, same order on both ranks
            models[r].exchange("send", nbytes, dsts=[1 - r])
            models[r].exchange("recv", nbytes, src=1 - r)
        stuck = simulate(_all(models))
        assert bool(stuck) == should_hang, (nbytes, stuck)


def test_simulate_reports_wrong_expectation():
    progs = {0: [Launch("k", pre=[(1, "c", 1)], waits=[("c", 2)])], 1: [Launch("k", pre=[(0, "c", 1)], waits=[("c", 1)])]}
    stuck = simulate(progs)
    assert len(stuck) == 1 and "rank 0" in stuck[0] and "c >= 2 (is 1)" in stuck[0]


def test_sync_monitor_matches_the_signature_and_names_divergence(monkeypatch):
    from mesh_b200.compiler import Program, compile_module, syncmon
    from mesh_b200.compiler.runtime import Executor, ThreadCollectives, ThreadWorld
    from mesh_b200.models.llama import Decoder, megatron
    monkeypatch.setenv("MESH_SYNC_TRACE", "1")
    torch.manual_seed(0)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1)
    x = torch.randn(1, 8, 32)
    procs = {"a": (0, "cpu"), "b": (0, "cpu")}
    names = tuple(procs)
    tp = megatron(procs)
    sch = compile_module(m, (x,), procs, lambda n: (1, names, None) if n.op == "placeholder" and n.name == "x" else tp(n))
    prog = Program(sch)                       # fused steps included: they log the collective they stand for
    # run rank by rank in threads, keeping the executors to read their traces
    import threading
    bound = prog.prepare((x,), {})
    world = ThreadWorld(2)
    exes = [Executor(prog.plan, r, ThreadCollectives(world, prog.mesh, r), torch.device("cpu")) for r in range(2)]
    ts = [threading.Thread(target=lambda e=e: e.run(bound, prog._consts)) for e in exes]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for e in exes:
        rep = syncmon.compare(sch, e.trace, prog.plan)
        assert rep["ok"] and rep["count_observed"] == rep["count_expected"] > 0, rep
    # without the fusion pass the executed order is the scheduled one and the digest is the compiled signature's
    assert syncmon.digest(sch, syncmon.expected(sch.plan)) == sch.signature.digest
    # a skipped collective and a swapped pair are named
    t = list(exes[0].trace)
    rep = syncmon.compare(sch, t[:3] + t[4:], prog.plan)
    assert not rep["ok"] and rep["first_divergence"]["index"] == 3 and len(rep["missing"]) == 1
    t[1], t[2] = t[2], t[1]
    rep = syncmon.compare(sch, t, prog.plan)
    assert not rep["ok"] and rep["first_divergence"]["index"] == 1 and rep["missing"] == []


def test_plans_with_fused_steps_pass_the_checker():
    """Fused (collective, product) pairs hand their gathered rows on under another name, and a ring step stands for the
    two gathers it replaced: the checker knows both."""
    import torch
    from mesh_b200.compiler import Program, check, compile_module
    from mesh_b200.models.llama import Decoder, megatron, sequence_parallel
    procs = {f"p{i}": (0, "cpu") for i in range(2)}
    names = tuple(procs)
    m = Decoder(dim=512, heads=4, ffn=1024, layers=1).eval()
    x = torch.randn(1, 256, 512)
    tp = megatron(procs)
    prog = Program(compile_module(m, (x,), procs, lambda nd: (1, names, None) if nd.op == "placeholder" and nd.name == "x" else tp(nd)))
    assert prog.fusion["ag_mm"] == 2 and check.check_plan(prog.plan) == []

    class Blocks(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.d = Decoder(dim=32, heads=4, ffn=64, layers=1)

        def forward(self, x):
            for b in self.d.blocks:
                x = b(x)
            return x
    prog = Program(compile_module(Blocks().eval(), (torch.randn(2, 12, 32),), procs, sequence_parallel(procs)))
    assert prog.fusion["ring_attention"] == 1 and check.check_plan(prog.plan) == []
