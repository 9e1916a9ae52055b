"""Processors on devices: crossing accounting, and a program interpreted with each processor on its own device."""
import pytest
import torch

from mesh_b200.compiler import Program, compile_module
from mesh_b200.compiler.devices import crossings, device_of, on_devices
from mesh_b200.models.llama import Decoder, megatron


def _model():
    torch.manual_seed(0)
    return Decoder(dim=32, heads=2, ffn=64, layers=1).eval(), torch.randn(2, 4, 32)


def test_crossings_count_transfers_between_machines():
    m, x = _model()
    far = {"a": (0, "cuda:0"), "b": (1, "cuda:0")}
    near = {"a": (0, "cuda:0"), "b": (0, "cuda:1")}
    sch = compile_module(m, (x,), far, megatron(far))
    rep = crossings(sch.plan, far)
    assert rep["transfers"] == len(sch.plan.transfers) > 0
    assert rep["between_machines"] == rep["transfers"] and rep["bytes_between_machines"] == sum(t.nbytes for t in sch.plan.transfers)
    assert set(rep["by_kind"]) == {"reduce"}
    rep = crossings(sch.plan, near)
    assert rep["between_machines"] == 0 and rep["between_devices"] == rep["transfers"]
    assert device_of((0, "cuda:1")) == torch.device("cuda", 1)
    if not torch.cuda.is_available():
        assert on_devices(far) == [torch.device("cpu")] * 2


def test_program_with_each_processor_on_its_device_matches_eager():
    m, x = _model()
    procs = {"a": (0, "cpu"), "b": (1, "cpu")}
    prog = Program(compile_module(m, (x,), procs, megatron(procs)), device="processors")
    assert prog.devices == [torch.device("cpu")] * 2
    assert torch.allclose(prog(x), m(x), atol=1e-5)


@pytest.mark.gpu
def test_gpu_and_host_processors_in_one_program():
    m, x = _model()
    procs = {"gpu": (0, "cuda:0"), "host": (0, "cpu")}
    prog = Program(compile_module(m, (x,), procs, megatron(procs)), device="processors", threads=True)
    assert [d.type for d in prog.devices] == ["cuda", "cpu"]
    out = prog(x)
    assert out.device.type == "cuda" and torch.allclose(out.cpu(), m(x), atol=1e-4)


def test_a_processor_that_is_an_engine_runs_its_products_on_the_host_engine():
    """Two processors: a torch device and the host engine.  The layers placed on the engine run as batches of the
    engine (products, the RMS norm, the residual sum), which reports the device that ran each; the result is the
    eager one."""
    import torch
    from mesh_b200.compiler import Program, compile_module
    from mesh_b200.models.llama import RMSNorm

    class Two(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = torch.nn.Linear(32, 64, bias=False), torch.nn.Linear(64, 32, bias=False)
            self.n = RMSNorm(32)

        def forward(self, x):
            h = torch.tanh(self.a(x))
            return x + self.b(h) + self.n(x)
    torch.manual_seed(0)
    m = Two().eval()
    x = torch.randn(8, 32)
    procs = {"dev": (0, "cpu"), "eng": (0, "host")}

    def placement(node):
        if node.op == "placeholder":
            return None
        return "dev" if node.name in ("mm", "tanh", "permute") else "eng"
    sch = compile_module(m, (x,), procs, placement)
    prog = Program(sch, device="processors", entry="eng")
    out = prog(x)
    assert torch.allclose(out, m(x), atol=1e-5)
    rep = prog.engine_report()
    kinds = {r["op"] for r in rep}
    assert "gemm_nt" in kinds and all(r["processor"] == "eng" and r["device"].startswith("cpu") for r in rep), rep
