"""lower(scheduled): per-processor programs agree with the interpreted plan and drop what a processor never touches."""
import threading

import torch

from mesh_b200.compiler import Program, compile_module
from mesh_b200.compiler.lower import lower
from mesh_b200.compiler.runtime import ThreadCollectives, ThreadWorld
from mesh_b200.models.llama import Decoder, megatron


def _run_lowered(sch, progs, x):
    prog = Program(sch)
    bound = prog.prepare((x,), {})
    world = ThreadWorld(len(progs))
    results = {}

    def work(name, p):
        results[name] = p.run(prog.plan, bound, prog._consts, ThreadCollectives(world, prog.mesh, p.rank))
    ts = [threading.Thread(target=work, args=(n, p)) for n, p in progs.items()]
    [t.start() for t in ts]
    [t.join() for t in ts]
    return prog, results


def test_lowered_spmd_program_matches_and_reads_well():
    torch.manual_seed(0)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1).eval()
    x = torch.randn(2, 4, 32)
    procs = {"a": (0, "cpu"), "b": (0, "cpu")}
    sch = compile_module(m, (x,), procs, megatron(procs))
    prog = Program(sch)
    progs = lower(sch, prog.plan)
    assert set(progs) == {"a", "b"}
    src = progs["a"].source
    assert src.startswith("def processor_a(") and "all_reduce(" in src and "mm.default(" in src and src.rstrip().endswith("]")
    _, results = _run_lowered(sch, progs, x)
    want = m(x)
    for r in results.values():
        assert torch.allclose(r[0], want, atol=1e-5)


def test_layers_on_different_processors_lower_to_different_programs():
    import sys, os
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples"))
    import importlib
    for mod in ("common", "engines"):
        sys.modules.pop(mod, None)
    eng = importlib.import_module("engines")
    torch.manual_seed(0)
    model = eng.Stack(32, 48, 4, "add").eval()
    x = torch.randn(8, 32)
    procs = {"p0": (0, "cpu"), "p1": (0, "cpu")}
    sch = compile_module(model, (x,), procs, eng.placement(tuple(procs)))
    prog = Program(sch)
    progs = lower(sch, prog.plan)
    n_all = len(prog.plan.steps)
    n0, n1 = len(progs["p0"].steps), len(progs["p1"].steps)
    assert n0 < n_all and n1 < n_all and n0 + n1 >= n_all - 2        # each processor only runs its own layers (+ transfers)
    assert "send_recv(" in progs["p0"].source and "send_recv(" in progs["p1"].source
    _, results = _run_lowered(sch, progs, x)
    want = model(x)
    got = [r[0] for r in results.values() if r[0] is not None]
    assert got and all(torch.allclose(g, want, atol=1e-4) for g in got)


def _run_generated(sch, plan, x):
    """Run the generated host programs of every processor on threads, as the lowered programs are run above."""
    from mesh_b200.compiler.hostgen import generate
    from mesh_b200.compiler.runtime import Executor
    prog = Program(sch)
    bound = prog.prepare((x,), {})
    hosts = generate(sch, plan)
    world = ThreadWorld(len(hosts))
    results = {}

    def work(name, hp):
        ex = Executor(plan, hp.rank, ThreadCollectives(world, prog.mesh, hp.rank), torch.device("cpu"))
        results[name] = hp.load()(ex, bound, prog._consts)
    ts = [threading.Thread(target=work, args=(n, h)) for n, h in hosts.items()]
    [t.start() for t in ts]
    [t.join() for t in ts]
    return hosts, results


def test_generated_host_programs_run_without_the_interpreter():
    """Every processor's steps as Python source that calls the operators directly (collectives and special steps
    through the executor): it compiles, most lines are direct calls, and the numbers are the interpreted plan's; a
    program with layers on different processors generates different functions, values elsewhere read as None."""
    torch.manual_seed(0)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1).eval()
    x = torch.randn(2, 4, 32)
    procs = {"a": (0, "cpu"), "b": (0, "cpu")}
    sch = compile_module(m, (x,), procs, megatron(procs))
    prog = Program(sch)
    hosts, results = _run_generated(sch, prog.plan, x)
    src = hosts["a"].source
    assert src.startswith("def run(ex, inputs, consts):") and "aten.mul.Tensor(" in src and "ex.collective(STEPS[" in src
    assert hosts["a"].direct > hosts["a"].through_executor > 0
    want = m(x)
    for r in results.values():
        assert torch.allclose(r[0], want, atol=1e-5)

    import sys, os
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples"))
    import importlib
    for mod in ("common", "engines"):
        sys.modules.pop(mod, None)
    eng = importlib.import_module("engines")
    model = eng.Stack(32, 48, 4, "add").eval()
    x2 = torch.randn(8, 32)
    procs2 = {"p0": (0, "cpu"), "p1": (0, "cpu")}
    sch2 = compile_module(model, (x2,), procs2, eng.placement(tuple(procs2)))
    prog2 = Program(sch2)
    hosts2, results2 = _run_generated(sch2, prog2.plan, x2)
    assert hosts2["p0"].source != hosts2["p1"].source
    got = [r[0] for r in results2.values() if r[0] is not None]
    assert got and all(torch.allclose(g, model(x2), atol=1e-4) for g in got)
