"""``mesh::attention`` / ``mesh::attention_backward``: attention as one differentiable operator of training graphs."""
import pytest
import torch
import torch.nn.functional as F

from mesh_b200.compiler import Program, attention_op, compile_module
from mesh_b200.models.llama import Decoder, megatron, sequence_parallel


@pytest.mark.parametrize("kv_heads,causal", [(4, True), (2, True), (1, False)])
def test_operator_and_its_backward_match_scaled_dot_product_attention(kv_heads, causal):
    torch.manual_seed(0)
    q = torch.randn(2, 4, 6, 8, requires_grad=True)
    k = torch.randn(2, kv_heads, 6, 8, requires_grad=True)
    v = torch.randn(2, kv_heads, 6, 8, requires_grad=True)
    w = torch.randn(2, 4, 6, 8)
    y = attention_op.substitute(q, k, v, is_causal=causal, enable_gqa=True)
    (y * w).sum().backward()
    mine = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    ref = F.scaled_dot_product_attention(q, k, v, is_causal=causal, enable_gqa=True)
    (ref * w).sum().backward()
    assert torch.allclose(y, ref, atol=2e-6)
    for a, t in zip(mine, (q, k, v)):
        assert torch.allclose(a, t.grad, atol=2e-6)


def test_queries_state_their_positions_in_the_whole_sequence():
    torch.manual_seed(1)
    q, k, v = (torch.randn(1, 2, 8, 4) for _ in range(3))
    full = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    block = torch.ops.mesh.attention(q[:, :, 4:], k, v, True, 0.5, 4, 1)[0]            # the second half of the queries
    assert torch.allclose(block, full[:, :, 4:], atol=1e-6)
    every_other = torch.ops.mesh.attention(q[:, :, 1::2], k, v, True, 0.5, 1, 2)[0]    # a round-robin share
    assert torch.allclose(every_other, full[:, :, 1::2], atol=1e-6)
    # a mask tensor or dropout: the plain formulation, same numbers
    mask = torch.tril(torch.ones(8, 8, dtype=torch.bool))
    assert torch.allclose(attention_op.substitute(q, k, v, attn_mask=mask), full, atol=1e-6)


def _run(m, x, procs, place):
    sch = compile_module(m, (x,), procs, place, loss=0)
    res = Program(sch)(x)
    for p in m.parameters():
        p.grad = None
    loss = m(x)
    loss.backward()
    assert abs(float(res.outputs.detach()) - float(loss.detach())) < 1e-5
    scale = max(float(p.grad.abs().max()) for p in m.parameters())
    for k, g in res.parameters.items():
        r = dict(m.named_parameters())[k].grad
        if g.shape != r.shape:
            r = r[tuple(slice(0, n) for n in g.shape)]
        assert (g - r).abs().max() <= 2e-5 * scale, k
    return sch


@pytest.mark.parametrize("n,units", [(2, None), (4, "striped"), (2, (3, 1))])
def test_training_plans_carry_one_attention_and_one_backward_per_layer(n, units, monkeypatch):
    torch.manual_seed(2)
    m = Decoder(dim=32, heads=4, ffn=64, layers=2)
    x = torch.randn(2, 8, 32)
    procs = {f"p{i}": (0, "cpu") for i in range(n)}
    # heads cut (Megatron): attention and its backward are local
    sch = _run(m, x, procs, megatron(procs))
    names = [str(st.target) for st in sch.plan.steps]
    assert names.count("mesh.attention.default") == 2 and names.count("mesh.attention_backward.default") == 2
    assert set(sch.structure["by_verb"]) == {"all_reduce"} and sch.structure["gathering_fallbacks"] == 0
    # queries cut along the sequence: they stay cut and state their rows; keys and values are gathered, their
    # gradients are partial sums
    x = torch.randn(1, 8, 32)                                  # (one sample: the token cut is the rows' outermost factor)
    sch = _run(m, x, procs, sequence_parallel(procs, units=units))
    att = [st for st in sch.plan.steps if str(st.target) == "mesh.attention.default"]
    assert len(att) == 2 and all("query_rows" in st.meta for st in att)
    assert sch.structure["gathering_fallbacks"] == 0 and sch.structure["by_verb"].get("all_gather", 0) >= 4
    fewer = len(sch.plan.steps)
    monkeypatch.setenv("MESH_ATTENTION_OP", "0")               # the plain expansion: same numbers, many more steps
    sch = _run(m, x, procs, sequence_parallel(procs, units=units))
    assert not any("mesh.attention" in str(st.target) for st in sch.plan.steps) and len(sch.plan.steps) > fewer


@pytest.mark.parametrize("n,units", [(2, None), (3, (3, 1, 2))])
def test_token_cut_survives_a_training_step_with_several_samples(n, units):
    """``[B, T, E]`` with B > 1 and the tokens cut: the capture merges the rows of every linear layer with the tokens
    outermost, so the activations stay cut through forward and backward products - queries keep their rows, weight
    gradients are partial sums over the processors' tokens (all-reduced), key / value gradients are reduce-scattered;
    nothing gathers an activation for want of a description."""
    torch.manual_seed(3)
    m = Decoder(dim=32, heads=4, ffn=64, layers=2)
    x = torch.randn(2, 8, 32)
    procs = {f"p{i}": (0, "cpu") for i in range(n)}
    sch = _run(m, x, procs, sequence_parallel(procs, units=units))
    att = [st for st in sch.plan.steps if str(st.target) == "mesh.attention.default"]
    assert len(att) == 2 and all("query_rows" in st.meta for st in att)
    verbs = sch.structure["by_verb"]
    assert verbs.get("reduce_scatter", 0) == 2 and verbs["all_reduce"] >= len(list(m.parameters()))
    gathered = [t.value for t in sch.plan.transfers if t.verb == "all_gather"]
    assert len(gathered) == 6                              # keys and values of two layers forward, the output, one loss term


@pytest.mark.parametrize("dim", [0, 1])
def test_attention_of_one_tensor_with_itself(dim):
    """``attention(h, h, h)``: one value is queries, keys and values at once, so it cannot be both cut (as queries) and
    whole (as keys) along the sequence - that axis gathers; a cut along the samples is local as ever."""
    import torch.nn as nn

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.l = nn.Linear(8, 8)

        def forward(self, x):
            h = self.l(x).view(2, 6, 2, 4).transpose(1, 2)
            return F.scaled_dot_product_attention(h, h, h, is_causal=True).pow(2).mean()
    torch.manual_seed(4)
    m, x = Net(), torch.randn(2, 6, 8)
    procs = {f"p{i}": (0, "cpu") for i in range(2)}
    names = tuple(procs)
    sch = _run(m, x, procs, lambda n: (dim, names, None) if n.name == "x" else None)
    assert ("all_gather" in sch.structure["by_verb"]) == (dim == 1)


def _sp_rank(rank, world, rdv):
    torch.manual_seed(6)
    m = Decoder(dim=32, heads=4, ffn=64, layers=1)
    x = torch.randn(2, 9, 32)
    procs = {f"p{i}": (0, "cpu") for i in range(world)}
    sch = compile_module(m, (x,), procs, sequence_parallel(procs, units=(4, 2, 3)), loss=0)
    prog = Program(sch)
    assert not prog.threads
    res = prog(x)                                          # one process per processor
    loss = m(x)
    loss.backward()
    assert abs(float(res.outputs.detach()) - float(loss.detach())) < 1e-5
    scale = max(float(p.grad.abs().max()) for p in m.parameters())
    for k, g in res.parameters.items():
        r = dict(m.named_parameters())[k].grad
        assert g.shape == r.shape and (g - r).abs().max() <= 2e-5 * scale, k


def test_sequence_parallel_training_between_processes():
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_sp_rank, 3, init_pg="gloo")
