"""The one-call interface: program(block, *examples) -> run, Placement / Shard records, save and load."""
import torch

from mesh_b200.compiler.legacy import Function, Placement, Shard, load, program
from mesh_b200.models.llama import Decoder


def test_program_runner_with_placement_records(tmp_path):
    torch.manual_seed(0)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1).eval()
    x = torch.randn(2, 6, 32)
    procs = {"a": (0, "cpu"), "b": (0, "cpu")}
    pl = Placement(mesh=tuple(procs), splits={"col": Shard(0), "row": Shard(1, (3, 1))},
                   nodes={"*wq_weight": "col", "*wk_weight": "col", "*wv_weight": "col", "*w1_weight": "col",
                          "*w3_weight": "col", "*wo_weight": "row", "*w2_weight": "row"})
    run = program(m, x, processors=procs, placement=pl, copies=2, horizon=1)
    assert run.signature.ok() and run.structure["by_kind"].get("reduce", 0) >= 2
    want = m(x)
    assert torch.allclose(run(), want, atol=1e-5)
    # fill the next input set in place, run again, the first set is untouched
    nxt = run.inputs()
    nxt[0].copy_(2 * x)
    assert torch.allclose(run(), m(2 * x), atol=1e-5)
    assert run.ended(0) and run.ended()
    assert torch.allclose(run.inputs()[0], x)                    # set 0 comes round again
    run.save(str(tmp_path))
    again = load(str(tmp_path))
    assert torch.allclose(again(x), want, atol=1e-5)
    assert again.signature.digest == run.signature.digest if hasattr(run.signature, "digest") else True


def test_function_leaves_are_compiled_once():
    torch.manual_seed(1)

    class Step(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.randn(16, 16) / 4)

        def forward(self, x):
            return torch.tanh(x @ self.w)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.work = Function(Step(), Placement(("a", "b"), {"*w": "cut"}, {"cut": Shard(1)}))

        def forward(self, x):
            for _ in range(4):
                x = self.work(x)
            return x

    b = Block().eval()
    x = torch.randn(3, 16)
    run = program(b, x, processors={"a": (0, "cpu"), "b": (0, "cpu")})
    assert run.structure["function_calls"] == {"work": 4}
    assert torch.allclose(run(), b(x), atol=1e-5)
