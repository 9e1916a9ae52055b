"""Programs of calls: dependence between calls, chain cover / outstanding width, commutativity of accumulating calls."""
import torch

from mesh_b200.compiler import compile_program
from mesh_b200.compiler import export as E
from mesh_b200.compiler.calls import Poly, analyse, commutes


class Acc(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.w = torch.nn.Parameter(torch.randn(4, 4))

    def forward(self, acc, x):
        return acc + x @ self.w


class Scale(torch.nn.Module):
    def forward(self, acc, x):
        return acc * 2 + x


class Affine(torch.nn.Module):
    def forward(self, acc, x):
        return (acc - x) / 2 + 3 * x - acc * 0.5 + acc                  # = acc + 2.5 x: commutes, after normalisation


class Prog(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.a, self.b, self.t = Acc(), Acc(), Scale()

    def forward(self, x, y):
        p = self.a(torch.zeros_like(x), x)
        p = self.a(p, y)                                                # a chain of two calls of a
        q = self.b(x, y)                                                # independent of the chain
        return self.t(p, q)


def test_polynomial_normal_form():
    a, b, c = (Poly.atom(k) for k in "abc")
    assert (a + b) * c == c * b + a * c
    assert (a - b) + b == a and not (a * b == a + b)
    assert (a + b) * (a - b) == a * a - b * b
    assert hash((a + b) * c) == hash(c * a + c * b)


def test_commutativity_of_accumulating_calls():
    x, y = torch.randn(2, 4), torch.randn(2, 4)
    assert commutes(E.export(Acc(), (x, y)), 0)                         # acc + f(x): order of the updates is free
    assert not commutes(E.export(Acc(), (x, y)), 1)                     # through the other input it is not
    assert not commutes(E.export(Scale(), (x, y)), 0)                   # 2 (2 r + x1) + x2 != 2 (2 r + x2) + x1
    assert commutes(E.export(Affine(), (x, y)), 0)


def test_call_analysis_of_a_program():
    torch.manual_seed(0)
    x, y = torch.randn(2, 4), torch.randn(2, 4)
    prog = Prog()
    exported, counts = E.calls(prog, (x, y), ["a", "b", "t"])
    assert counts == {"a": 2, "b": 1, "t": 1}
    an = analyse(exported, ["a", "b", "t"], bodies={"a": E.export(Acc(), (x, y))})
    assert [f for f, _ in an.calls] == ["a", "a", "b", "t"]
    assert an.edges == [(0, 1), (1, 3), (2, 3)]
    assert an.closure[3] == {0, 1, 2} and an.closure[2] == set()
    assert an.width == 2 and an.chains[0] == an.chains[1] != an.chains[2]
    assert an.widths == {"a": 1, "b": 1, "t": 1} and an.outstanding("a") == 1
    s = an.summary()
    assert s["critical_path"] == ["a#0", "a#1", "t#0"] and s["commuting"]["a"] == {0: True, 1: False}


def test_compile_program_reports_the_analysis():
    torch.manual_seed(1)
    x, y = torch.randn(2, 4), torch.randn(2, 4)
    procs = {"p0": (0, "cpu"), "p1": (0, "cpu")}
    names = tuple(procs)
    sch = compile_program(Prog(), (x, y), ["a", "b", "t"], procs,
                          lambda node: (0, names, None) if node.op == "placeholder" and node.name in ("x", "y") else None)
    rep = sch.structure["call_analysis"]
    assert rep["calls"] == 4 and rep["width"] == 2 and sch.structure["function_calls"] == {"a": 2, "b": 1, "t": 1}


def test_substitute_replaces_every_call_of_a_function_by_its_parts():
    """A block function replaced by two parts that take over its parameters: same numbers, the parts are call
    instances of their own in the captured program, and the program still compiles and runs cut over two processors."""
    import torch

    from mesh_b200.compiler import calls as C
    from mesh_b200.compiler.export import Parts, calls, substitute

    class Block(torch.nn.Module):
        def __init__(self, d):
            super().__init__()
            self.lin = torch.nn.Linear(d, d)

        def forward(self, x, gate):
            return torch.tanh(self.lin(x)) * gate, x

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = Block(16), Block(16)

        def forward(self, x, gate):
            y, _ = self.a(x, gate)
            z, skip = self.b(y, gate)
            return z + skip

    class Project(torch.nn.Module):
        def __init__(self, lin):
            super().__init__()
            self.lin = lin

        def forward(self, x):
            return self.lin(x)

    class Gate(torch.nn.Module):
        def forward(self, h, gate):
            return torch.tanh(h) * gate

    torch.manual_seed(0)
    net = Net()
    x, gate = torch.randn(4, 16), torch.randn(4, 16)
    want = net(x, gate)
    n = substitute(net, Block, [("project", lambda blk: Project(blk.lin), [("call", 0)]),
                                ("gate", lambda blk: Gate(), [("part", 0, 0), ("call", 1)])],
                   results=[(1, 0), (0, 0)])
    assert n == 2 and isinstance(net.a, Parts) and isinstance(net.b, Parts)
    # output 1 of the original call was x itself; the substitution's second result is the projection instead, so the
    # network's skip term changes on purpose: state what it must be
    h1 = torch.tanh(net.a.project(x)) * gate
    lin2 = net.b.project(h1)
    assert torch.allclose(net(x, gate), torch.tanh(lin2) * gate + lin2, atol=1e-6)
    assert not torch.allclose(net(x, gate), want)
    # results that keep the original meaning: the pass-through output comes straight from the call's input
    net2 = Net()
    net2.load_state_dict({k.replace(".project.lin.", ".lin."): v for k, v in net.state_dict().items()})
    want2 = net2(x, gate)

    class Pass(torch.nn.Module):
        def forward(self, x):
            return x
    substitute(net2, Block, [("project", lambda blk: Project(blk.lin), [("call", 0)]),
                             ("gate", lambda blk: Gate(), [("part", 0, 0), ("call", 1)]),
                             ("keep", lambda blk: Pass(), [("call", 0)])], results=[(1, 0), (2, 0)])
    assert torch.allclose(net2(x, gate), want2, atol=1e-6)
    exp, counts = calls(net2, (x, gate), ["a.project", "a.gate", "b.project", "b.gate"])
    assert counts == {"a.project": 1, "a.gate": 1, "b.project": 1, "b.gate": 1}
    an = C.analyse(exp, ["a.project", "a.gate", "b.project", "b.gate"])
    assert len(an.calls) == 4
