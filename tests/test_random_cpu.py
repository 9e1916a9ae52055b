"""Random draws in compiled programs do not depend on how the tensors are cut (counter-based generator, draw sites)."""
import torch

from mesh_b200.compiler import Program, compile_module


class Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.fc, self.fc2 = torch.nn.Linear(8, 8), torch.nn.Linear(8, 8)

    def forward(self, x):
        h = torch.nn.functional.dropout(self.fc(x), 0.25, training=True)
        h = self.fc2(h) * torch.rand_like(h) + 0.1 * torch.randn_like(h) + torch.bernoulli(torch.full_like(h, 0.5))
        return (h * h).mean()


def _run(n, m, x, seed=1234, calls=2):
    procs = {f"p{i}": (0, "cpu") for i in range(n)}
    names = tuple(procs)

    def placement(node):
        if node.op != "placeholder":
            return None
        if node.name == "x":
            return (0, names, None)
        if "fc2_weight" in node.name:
            return (1, names, None)                                   # partial sums meet a draw
        return None
    sch = compile_module(m, (x,), procs, placement, loss=0)
    prog = Program(sch)
    prog.seed = seed
    return sch, [prog(x) for _ in range(calls)]


def test_draws_are_the_same_on_one_two_and_four_processors():
    torch.manual_seed(0)
    m, x = Net(), torch.randn(8, 8)
    sch1, one = _run(1, m, x)
    assert [st.meta["site"] for st in sch1.plan.steps if "draw" in st.meta] == [0, 1, 2, 3]
    assert abs(float(one[0].outputs) - float(one[1].outputs)) > 1e-4        # the next execution draws fresh numbers
    for n in (2, 4):
        sch, many = _run(n, m, x)
        assert sch.structure["fallbacks"] == 0
        for a, b in zip(one, many):
            assert abs(float(a.outputs) - float(b.outputs)) < 1e-5
            assert torch.allclose(a.parameters["fc.weight"], b.parameters["fc.weight"], atol=1e-5)
            assert torch.allclose(a.parameters["fc.bias"], b.parameters["fc.bias"], atol=1e-5)
    _, other = _run(2, m, x, seed=99, calls=1)
    assert abs(float(other[0].outputs) - float(one[0].outputs)) > 1e-4      # another seed, other numbers


def test_dropout_rate_and_normal_moments():
    class Draws(torch.nn.Module):
        def forward(self, x):
            return torch.nn.functional.dropout(x, 0.3, training=True), torch.randn_like(x), torch.rand_like(x)

    x = torch.ones(64, 512)
    procs = {"p0": (0, "cpu"), "p1": (0, "cpu")}
    names = tuple(procs)
    sch = compile_module(Draws(), (x,), procs, lambda node: (1, names, "striped") if node.name == "x" else None)
    dropped, normal, uniform = Program(sch)(x)
    kept = (dropped != 0).float().mean()
    assert abs(float(kept) - 0.7) < 0.01 and torch.allclose(dropped[dropped != 0], torch.tensor(1 / 0.7))
    assert abs(float(normal.mean())) < 0.02 and abs(float(normal.std()) - 1) < 0.02
    assert abs(float(uniform.mean()) - 0.5) < 0.01 and 0 <= float(uniform.min()) and float(uniform.max()) < 1
