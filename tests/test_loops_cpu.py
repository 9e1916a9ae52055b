"""``map`` and ``scan`` higher-order operators are unrolled at capture, then placed like any other graph."""
import torch
from torch._higher_order_ops.map import map as hop_map
from torch._higher_order_ops.scan import scan

from mesh_b200.compiler import Program, compile_module
from mesh_b200.compiler import export as E


class Recurrent(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.w = torch.nn.Parameter(torch.randn(4, 4) * 0.3)

    def forward(self, xs, h0):
        ys = hop_map(lambda x, w: torch.tanh(x @ w), xs, self.w)

        def step(h, x):
            h2 = torch.tanh(h @ self.w + x)
            return h2, h2 * 2
        return scan(step, h0, ys)


class Loss(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.m = Recurrent()

    def forward(self, xs, h0):
        last, out = self.m(xs, h0)
        return (last * last).mean() + out.mean()


def _by_hand(w, xs, h0):
    ys = torch.tanh(xs @ w)
    h, outs = h0, []
    for i in range(xs.shape[0]):
        h = torch.tanh(h @ w + ys[i])
        outs.append(2 * h)
    return h, torch.stack(outs)


def _placement(names):
    def placement(node):
        if node.op != "placeholder":
            return None
        return (1, names, None) if node.name == "xs" else (0, names, None) if node.name == "h0" else None
    return placement


def test_capture_has_no_loop_operators_left():
    torch.manual_seed(0)
    ex = E.export(Recurrent(), (torch.randn(5, 6, 4), torch.randn(6, 4)))
    targets = [n.target for n in ex.graph_module.graph.nodes if n.op == "call_function"]
    assert not [t for t in targets if "higher_order" in str(t)]
    assert sum(t is torch.ops.aten.tanh.default for t in targets) == 5 + 5       # one map body and one scan body per step


def test_unrolled_loops_over_a_batch_cut_inference_and_training():
    torch.manual_seed(0)
    xs, h0 = torch.randn(5, 6, 4), torch.randn(6, 4)
    procs = {"p0": (0, "cpu"), "p1": (0, "cpu")}
    m = Recurrent()
    sch = compile_module(m, (xs, h0), procs, _placement(tuple(procs)))
    assert sch.structure["fallbacks"] == 0 and sch.structure["by_verb"] == {"all_gather": 2}    # only the two results
    last, out = Program(sch)(xs, h0)
    ref_last, ref_out = _by_hand(m.w.detach(), xs, h0)
    assert torch.allclose(last, ref_last, atol=1e-6) and torch.allclose(out, ref_out, atol=1e-6)
    net = Loss()
    res = Program(compile_module(net, (xs, h0), procs, _placement(tuple(procs)), loss=0))(xs, h0)
    w = net.m.w.detach().clone().requires_grad_(True)
    h, o = _by_hand(w, xs, h0)
    loss = (h * h).mean() + o.mean()
    loss.backward()
    assert abs(float(res.outputs) - float(loss)) < 1e-6
    assert torch.allclose(res.parameters["m.w"], w.grad, atol=1e-6)


def test_archive_round_trip_of_a_program_with_unrolled_loops(tmp_path):
    from mesh_b200.compiler import archive
    torch.manual_seed(2)
    xs, h0 = torch.randn(5, 6, 4), torch.randn(6, 4)
    procs = {"p0": (0, "cpu"), "p1": (0, "cpu")}
    sch = compile_module(Recurrent(), (xs, h0), procs, _placement(tuple(procs)))
    archive.save(tmp_path / "a", sch)
    back = archive.load(tmp_path / "a")
    assert back.signature.digest == sch.signature.digest
    a, b = Program(sch)(xs, h0), Program(back)(xs, h0)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
