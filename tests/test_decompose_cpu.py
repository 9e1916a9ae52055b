"""Source formulations of linear-algebra operators: numerics against torch.linalg, capture, and a batch cut."""
import collections

import pytest
import torch

from mesh_b200.compiler import Program, compile_module, decompose
from mesh_b200.models.llama import data_parallel


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-9), (torch.float32, 2e-4)])
def test_formulations_match_the_library(dtype, tol):
    torch.manual_seed(0)
    a = torch.randn(3, 9, 9, dtype=dtype)
    ref = torch.linalg.matrix_exp(a)
    assert (decompose.matrix_exp(a) - ref).abs().max() <= tol * ref.abs().max()
    big = 20 * a                                                        # needs several squarings
    ref = torch.linalg.matrix_exp(big)
    assert (decompose.matrix_exp(big) - ref).abs().max() <= 100 * tol * ref.abs().max()
    t = torch.randn(3, 12, 9, dtype=dtype)
    u, h = decompose.polar(t)
    eye = torch.eye(9, dtype=dtype)
    assert (u @ h - t).abs().max() < tol and (u.mT @ u - eye).abs().max() < tol
    assert torch.linalg.eigvalsh(h).min() > -tol
    sym = a + a.mT
    w, v = decompose.eigh(sym)
    assert (w - torch.linalg.eigvalsh(sym)).abs().max() < tol * 10
    assert (v @ torch.diag_embed(w) @ v.mT - sym).abs().max() < tol * 10 and (v.mT @ v - eye).abs().max() < tol
    for m in (t, t.mT):
        U, S, Vh = decompose.svd(m)
        assert (S - torch.linalg.svdvals(m)).abs().max() < tol * 10
        assert (U @ torch.diag_embed(S) @ Vh - m).abs().max() < tol * 10
    low = t[..., :4] @ torch.randn(3, 4, 9, dtype=dtype)              # rank 4
    rtol = 1e-5 if dtype == torch.float32 else 1e-12
    assert (decompose.pinv(low, rtol=rtol) - torch.linalg.pinv(low, rtol=rtol)).abs().max() < tol
    b = torch.randn(3, 12, 2, dtype=dtype)
    assert (decompose.lstsq(t, b) - torch.linalg.lstsq(t, b).solution).abs().max() < tol


@pytest.mark.parametrize("n", [1, 2, 5])
def test_eigh_small_and_odd_sizes(n):
    torch.manual_seed(n)
    a = torch.randn(2, n, n, dtype=torch.float64)
    sym = a + a.mT
    w, v = decompose.eigh(sym)
    assert (w - torch.linalg.eigvalsh(sym)).abs().max() < 1e-12
    assert (v @ torch.diag_embed(w) @ v.mT - sym).abs().max() < 1e-12


class _Linalg(torch.nn.Module):
    def forward(self, x):
        return (torch.linalg.matrix_exp(0.3 * x), torch.linalg.eigh(x + x.mT)[0], torch.linalg.pinv(x),
                torch.linalg.svd(x, full_matrices=False)[1])


def test_capture_expands_the_operators_and_a_batch_cut_stays_local():
    torch.manual_seed(1)
    m, x = _Linalg(), torch.randn(4, 6, 6)
    procs = {"p0": (0, "cpu"), "p1": (0, "cpu")}
    sch = compile_module(m, (x,), procs, data_parallel(procs), decompositions=decompose.table(max_squarings=4))
    targets = {st.target for st in sch.plan.steps if st.op == "call"}
    assert not targets & set(decompose.EXPANDED)
    assert not [st for st in sch.plan.steps if st.meta.get("fallback")]
    # the only transfers bring the four results together
    assert collections.Counter(st.target for st in sch.plan.steps if st.op == "collective") == {"all_gather": 4}
    out = Program(sch)(x)
    for got, ref in zip(out, m(x)):
        assert (got - ref).abs().max() < 2e-4 * max(1.0, float(ref.abs().max()))


def test_training_batch_norm_under_a_batch_cut_uses_whole_batch_statistics():
    import copy

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c, self.bn = torch.nn.Conv2d(4, 4, 3, padding=1), torch.nn.BatchNorm2d(4)

        def forward(self, x):
            return (x + torch.relu(self.bn(self.c(x)))).pow(2).mean()

    torch.manual_seed(2)
    m, x = Net(), torch.randn(4, 4, 8, 8)
    ref = copy.deepcopy(m)
    procs = {"p0": (0, "cpu"), "p1": (0, "cpu")}
    sch = compile_module(m, (x,), procs, data_parallel(procs), loss=0, decompositions=decompose.norms())
    assert sch.structure["fallbacks"] == 0 and "all_gather" not in sch.structure["by_verb"]
    res = Program(sch)(x)
    loss = ref(x)
    loss.backward()
    assert abs(float(res.outputs) - float(loss)) < 1e-6
    for k, p in ref.named_parameters():
        assert torch.allclose(res.parameters[k], p.grad, atol=1e-5), k
    # the running statistics were stored into the module's own buffers, once
    assert torch.allclose(m.bn.running_mean, ref.bn.running_mean, atol=1e-6)
    assert torch.allclose(m.bn.running_var, ref.bn.running_var, atol=1e-6)
    assert int(m.bn.num_batches_tracked) == int(ref.bn.num_batches_tracked) == 1
