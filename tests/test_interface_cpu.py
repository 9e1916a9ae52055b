"""The program interface: output pytrees, keyword inputs, buffer and input mutations, integer inputs, loss position."""
import torch

from mesh_b200.compiler import Program, compile_module

PROCS = {"p0": (0, "cpu"), "p1": (0, "cpu")}
NAMES = tuple(PROCS)


def _cut0(*which):
    return lambda nd: (0, NAMES, None) if nd.op == "placeholder" and nd.name in which else None


def _data():
    g = torch.Generator().manual_seed(0)
    return torch.randn(4, 3, generator=g), torch.randn(4, 3, generator=g)


def test_output_pytrees_and_keyword_inputs():
    class Tree(torch.nn.Module):
        def forward(self, x, y):
            return {"s": x + y, "p": (x * y).sum(0), "n": [x.mean(), y.amax()]}

    class Kw(torch.nn.Module):
        def forward(self, x, *, y, scale=2.0):
            return x * scale + y

    x, y = _data()
    out = Program(compile_module(Tree(), (x, y), PROCS, _cut0("x", "y")))(x, y)
    ref = Tree()(x, y)
    assert torch.allclose(out["s"], ref["s"]) and torch.allclose(out["p"], ref["p"], atol=1e-6)
    assert torch.allclose(out["n"][0], ref["n"][0], atol=1e-6) and torch.allclose(out["n"][1], ref["n"][1])
    out = Program(compile_module(Kw(), (x,), PROCS, _cut0("x", "y"), kwargs={"y": y}))(x, y=y)
    assert torch.allclose(out, 2 * x + y)


def test_buffer_and_input_mutations_are_stored_in_place():
    class Counter(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.register_buffer("steps", torch.zeros(()))
            self.register_buffer("ema", torch.zeros(3))

        def forward(self, x):
            self.steps += 1
            self.ema.mul_(0.9).add_(x.mean(0) * 0.1)
            return x - self.ema

    class Doubles(torch.nn.Module):
        def forward(self, x):
            x.mul_(2)
            return x.sum(0)

    x, _ = _data()
    m, ref = Counter(), Counter()
    prog = Program(compile_module(m, (x,), PROCS, _cut0("x")))
    for step in (1, 2):                                                  # the buffers carry over between calls
        assert torch.allclose(prog(x), ref(x), atol=1e-6)
        assert float(m.steps) == step and torch.allclose(m.ema, ref.ema, atol=1e-6)
    mine = x.clone()
    out = Program(compile_module(Doubles(), (mine,), PROCS, _cut0("x")))(mine)
    assert torch.allclose(out, (2 * x).sum(0), atol=1e-6) and torch.allclose(mine, 2 * x)      # the caller's tensor changed


def test_integer_inputs_in_place_arithmetic_and_loss_position():
    class Lookup(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.e = torch.nn.Embedding(10, 4)

        def forward(self, idx, mask):
            return (self.e(idx) * mask[..., None]).sum(1)

    class Inplace(torch.nn.Module):
        def forward(self, x):
            z = x.clone()
            z[:, 0] = 0
            z.add_(1).clamp_(max=1.5)
            z[1:3] *= 2
            return z

    class TwoOutputs(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.l = torch.nn.Linear(3, 2)

        def forward(self, x):
            h = self.l(x)
            return h.detach().abs().max(), h.pow(2).mean()               # a monitored value, then the loss

    torch.manual_seed(1)
    x, _ = _data()
    idx, mask = torch.randint(0, 10, (4, 5)), torch.rand(4, 5) > 0.3
    m = Lookup()
    assert torch.allclose(Program(compile_module(m, (idx, mask), PROCS, _cut0("idx", "mask")))(idx, mask), m(idx, mask), atol=1e-6)
    assert torch.allclose(Program(compile_module(Inplace(), (x,), PROCS, _cut0("x")))(x), Inplace()(x))
    m = TwoOutputs()
    res = Program(compile_module(m, (x,), PROCS, _cut0("x"), loss=1))(x)
    aux, loss = m(x)
    loss.backward()
    assert torch.allclose(res.outputs[0], aux) and torch.allclose(res.outputs[1], loss)
    assert torch.allclose(res.parameters["l.weight"], m.l.weight.grad, atol=1e-6)
