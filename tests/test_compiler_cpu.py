"""Sharding compiler end to end on CPU (threads executor = every processor in one process):
compiled forward+backward vs eager PyTorch, for TP / DP / SP / striped CP / unequal shards / 2-D meshes."""
import pytest
import torch

from mesh_b200.compiler import Program, compile_module, counts
from mesh_b200.models.llama import Decoder, data_parallel, megatron, sequence_parallel


def _procs(n):
    return {f"p{i}": (0, "cpu") for i in range(n)}


def _eager(m, x):
    for p in m.parameters():
        p.grad = None
    loss = m(x)
    loss.backward()
    return loss.detach(), {k: p.grad.clone() for k, p in m.named_parameters()}


def _check(res, loss, grads, plan=None, rank=0, tol=2e-5):
    assert abs(float(res.outputs) - float(loss)) < tol * max(1.0, abs(float(loss)))
    for k, g in res.parameters.items():
        ref = grads[k]
        if g.shape != ref.shape:            # sharded parameter: rank 0 holds the first block
            sl = tuple(slice(0, s) for s in g.shape)
            ref = ref[sl]
        assert (g - ref).abs().max() <= tol * (ref.abs().max() + 1e-6) + 1e-7, k


@pytest.mark.parametrize("n", [2, 4])
def test_tensor_parallel_block(n):
    torch.manual_seed(0)
    m = Decoder(dim=64, heads=4, ffn=128, layers=2)
    x = torch.randn(2, 8, 64)
    procs = _procs(n)
    sch = compile_module(m, (x,), procs, megatron(procs), loss=0)
    assert sch.signature.ok() and sch.structure["by_kind"].get("reduce", 0) >= 4
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


def test_data_parallel_gradients_all_reduce():
    torch.manual_seed(1)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1)
    x = torch.randn(4, 6, 32)
    procs = _procs(2)
    sch = compile_module(m, (x,), procs, data_parallel(procs), loss=0)
    assert sch.structure["by_verb"].get("all_reduce", 0) >= len(list(m.parameters()))
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


@pytest.mark.parametrize("units", [None, "striped", (3, 1)])
def test_sequence_sharding_causal_attention(units):
    torch.manual_seed(2)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1)
    x = torch.randn(2, 12, 32)
    procs = _procs(2)
    sch = compile_module(m, (x,), procs, sequence_parallel(procs, units=units), loss=0)
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads, tol=5e-5)


def test_unequal_shards_and_counts():
    assert counts(10, None, 4) == [3, 3, 3, 1]                       # torch.chunk sizes
    assert counts(10, "striped", 4) == [3, 3, 2, 2]
    assert counts(16, (11904, 3456), 2) == [12, 4]                   # the reference's Goal A split ratio
    assert sum(counts(4096, (7, 1, 3), 3)) == 4096
    assert counts(10, (0, 4, 10), 2) == [4, 6]                       # explicit edges
    torch.manual_seed(3)
    m = Decoder(dim=64, heads=4, ffn=96, layers=1)
    x = torch.randn(2, 4, 64)
    procs = _procs(2)
    sch = compile_module(m, (x,), procs, megatron(procs, units=(3, 1)), loss=0)
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)
    assert res.parameters["blocks.0.w1.weight"].shape[0] == 72       # 3/4 of 96 rows on processor 0


def test_two_dimensional_mesh_dp_x_tp():
    torch.manual_seed(4)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1)
    x = torch.randn(4, 4, 32)
    procs = _procs(4)
    tp = megatron(procs)

    def placement(node):
        if node.op != "placeholder":
            return None
        if node.name == "x":
            return ((0, None), None, (None, None))                     # batch over mesh axis 0
        st = tp(node)
        if st is None:
            return None
        return ((None, st[0]), None, (None, None))                     # weights over mesh axis 1
    sch = compile_module(m, (x,), procs, placement, loss=0, mesh=(2, 2))
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


def test_inference_output_and_structure_report():
    torch.manual_seed(5)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1)
    x = torch.randn(2, 4, 32)
    procs = _procs(2)
    sch = compile_module(m, (x,), procs, megatron(procs))
    out = Program(sch)(x)
    assert torch.allclose(out, m(x), atol=1e-5)
    s = sch.structure
    assert s["uncovered"] == 0 and s["unwaited"] == 0 and s["channels"] == sum(s["by_kind"].values())


def test_archive_round_trip(tmp_path):
    from mesh_b200.compiler import archive
    torch.manual_seed(6)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1)
    x = torch.randn(2, 4, 32)
    procs = _procs(2)
    sch = compile_module(m, (x,), procs, megatron(procs), loss=0)
    archive.save(tmp_path / "a", sch)
    back = archive.load(tmp_path / "a")
    assert back.signature.digest == sch.signature.digest
    r0, r1 = Program(sch)(x), Program(back)(x)
    assert torch.equal(r0.outputs, r1.outputs)
    for k in r0.parameters:
        assert torch.equal(r0.parameters[k], r1.parameters[k])


def _dist_rank(rank, world, rdv):
    import torch.distributed as dist
    torch.manual_seed(7)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1)
    x = torch.randn(2, 6, 32)
    procs = _procs(world)
    sch = compile_module(m, (x,), procs, megatron(procs), loss=0)
    res = Program(sch)(x)                      # distributed executor: this process is processor `rank`
    loss, grads = _eager(m, x)
    assert abs(float(res.outputs) - float(loss)) < 1e-5
    g = res.parameters["blocks.0.w1.weight"]
    rows = g.shape[0]
    ref = grads["blocks.0.w1.weight"][rank * rows:(rank + 1) * rows]
    assert (g - ref).abs().max() < 1e-5 * (ref.abs().max() + 1e-6) + 1e-7


def test_program_distributed_gloo():
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_dist_rank, 2, init_pg="gloo")


@pytest.mark.parametrize("n,dim", [(2, 2), (4, 3)])
def test_convolution_with_halo_exchange(n, dim):
    """A 'same' convolution over an input cut along a spatial dimension: neighbours exchange edge rows."""
    torch.manual_seed(7)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c1 = torch.nn.Conv2d(3, 8, 3, padding=1)
            self.c2 = torch.nn.Conv2d(8, 4, 5, padding=4, dilation=2)

        def forward(self, x):
            return self.c2(torch.relu(self.c1(x)))

    m = Net().eval()
    x = torch.randn(2, 3, 16, 16)
    procs = _procs(n)
    names = tuple(procs)
    sch = compile_module(m, (x,), procs, lambda node: (dim, names, None) if node.op == "placeholder" and node.name == "x" else None)
    verbs = sch.structure["by_verb"]
    assert verbs.get("halo", 0) == 2 and verbs.get("all_gather", 0) == 1, verbs      # two exchanges, one gather of the result
    out = Program(sch)(x)
    assert torch.allclose(out, m(x), atol=1e-5)


def test_collective_matmul_pairs_are_fused_and_results_unchanged(monkeypatch):
    """Sequence-parallel Megatron block: the all-gather -> mm and mm -> reduce-scatter pairs become fused steps
    (run unfused on CPU ranks), and the program computes what it computed before the rewrite."""
    torch.manual_seed(8)
    m = Decoder(dim=64, heads=4, ffn=128, layers=2)
    x = torch.randn(1, 16, 64)
    procs = _procs(2)
    names = tuple(procs)
    tp = megatron(procs)

    def placement(node):
        if node.op == "placeholder" and node.name == "x":
            return (1, names, None)
        return tp(node)
    sch = compile_module(m, (x,), procs, placement, loss=0)
    prog = Program(sch)
    assert prog.fusion["ag_mm"] >= 4 and prog.fusion["mm_rs"] >= 2, prog.fusion
    assert any(st.op == "fused" for st in prog.plan.steps)
    res = prog(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads, tol=5e-5)
    monkeypatch.setenv("MESH_FUSE", "0")
    plain = Program(sch)
    assert plain.fusion == {"ag_mm": 0, "mm_rs": 0}
    res2 = plain(x)
    assert abs(float(res2.outputs) - float(res.outputs)) < 1e-6


def test_plan_cache_hits_and_key_sensitivity(tmp_path):
    import time
    from mesh_b200.compiler.cache import cache_key, compile_cached
    torch.manual_seed(9)
    m = Decoder(dim=32, heads=2, ffn=64, layers=1).eval()
    x = torch.randn(2, 4, 32)
    procs = _procs(2)
    t0 = time.perf_counter()
    sch, hit = compile_cached(m, (x,), procs, megatron(procs), tmp_path)
    t_miss = time.perf_counter() - t0
    assert not hit
    t0 = time.perf_counter()
    sch2, hit2 = compile_cached(m, (x,), procs, megatron(procs), tmp_path)
    t_hit = time.perf_counter() - t0
    assert hit2 and t_hit < t_miss
    assert torch.allclose(Program(sch2)(x), m(x), atol=1e-5)
    k0 = cache_key(m, (x,), procs, megatron(procs))
    assert k0 == cache_key(m, (x,), procs, megatron(procs))
    assert k0 != cache_key(m, (torch.randn(2, 8, 32),), procs, megatron(procs))             # other shapes
    assert k0 != cache_key(m, (x,), _procs(4), megatron(_procs(4)))                           # other processors
    assert k0 != cache_key(m, (x,), procs, megatron(procs, units=(3, 1)))                     # other shares
    assert k0 != cache_key(m, (x,), procs, megatron(procs), loss=0)                           # other options
    assert k0 != cache_key(Decoder(dim=32, heads=2, ffn=96, layers=1), (x,), procs, megatron(procs))


def test_observed_step_times():
    from mesh_b200.compiler.observe import observe, stage_costs
    torch.manual_seed(10)
    m = Decoder(dim=64, heads=4, ffn=256, layers=2).eval()
    x = torch.randn(2, 16, 64)
    procs = _procs(2)
    prog = Program(compile_module(m, (x,), procs, megatron(procs)))
    rep = observe(prog, x, repeats=2)
    assert len(rep["steps"]) == len(prog.plan.steps) and rep["total"] > 0
    assert any(k.startswith("blocks.1") for k in rep["by_module"]) and rep["by_kind"].get("collective", 0) > 0
    stages = stage_costs(rep, prog.plan)
    n_coll = sum(1 for st in prog.plan.steps if st.op == "collective" or (st.op == "fused" and "channel" in st.meta))
    assert len(stages) in (n_coll, n_coll + 1)
    assert abs(sum(s["compute_s"] + s["collective_s"] for s in stages) - rep["total"]) < 1e-9
    # observation is off again afterwards
    prog(x)
    assert prog.per_rank[0][0].times is None


def test_attention_stays_whole_when_heads_are_cut():
    """Inference graphs keep attention as one operation; with the heads cut over processors it needs no transfer."""
    class Attn(torch.nn.Module):
        def __init__(self, dim, heads):
            super().__init__()
            self.heads = heads
            self.wq, self.wk, self.wv, self.wo = (torch.nn.Linear(dim, dim, bias=False) for _ in range(4))

        def forward(self, x):
            B, T, D = x.shape
            split = lambda t: t.view(B, T, self.heads, D // self.heads).transpose(1, 2)
            o = torch.nn.functional.scaled_dot_product_attention(split(self.wq(x)), split(self.wk(x)), split(self.wv(x)),
                                                                 is_causal=True)
            return self.wo(o.transpose(1, 2).reshape(B, T, D))

    torch.manual_seed(11)
    m = Attn(32, 4).eval()
    x = torch.randn(2, 8, 32)
    procs = _procs(2)

    names = tuple(procs)

    def placement(node):
        if node.op != "placeholder":
            return None
        if any(k in node.name for k in ("wq", "wk", "wv")):
            return (0, names, None)                                   # rows = heads
        if "wo" in node.name:
            return (1, names, None)
        return None
    sch = compile_module(m, (x,), procs, placement)
    targets = [str(st.target) for st in sch.plan.steps if st.op == "call"]
    assert any("scaled_dot_product_attention" in t for t in targets)
    assert [st.target for st in sch.plan.steps if st.op == "collective"] == ["all_reduce"]
    assert torch.allclose(Program(sch)(x), m(x), atol=1e-5)


def test_batched_operators_with_several_outputs_keep_a_batch_cut():
    """Layer norm (forward and backward) and sort over a batch cut: no gathers, weight gradients are partial sums."""
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ln, self.fc = torch.nn.LayerNorm(16), torch.nn.Linear(16, 8)

        def forward(self, x):
            values, _ = torch.sort(self.fc(self.ln(x)), dim=-1)
            return (values * values).mean()

    torch.manual_seed(12)
    m, x = Net(), torch.randn(4, 6, 16)
    procs = _procs(2)
    sch = compile_module(m, (x,), procs, data_parallel(procs), loss=0)
    assert not [st for st in sch.plan.steps if st.meta.get("fallback")]
    assert {st.target for st in sch.plan.steps if st.op == "collective"} == {"all_reduce"}
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


class _ConvNet(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.c1, self.c2 = torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.Conv2d(8, 8, 5, padding=2)
        self.fc = torch.nn.Linear(8 * 4 * 4, 5)

    def forward(self, x):
        h = torch.nn.functional.max_pool2d(torch.relu(self.c1(x)), 2)
        h = torch.nn.functional.avg_pool2d(torch.relu(self.c2(h)), 2)
        return self.fc(h.flatten(1)).pow(2).mean()


@pytest.mark.parametrize("n,dim", [(2, 2), (2, 3), (2, 0)])
def test_convolution_network_trains_under_a_spatial_or_batch_cut(n, dim):
    """Convolution forward and backward with halo exchange (and its adjoint), pooling whose windows do not straddle a
    cut, and the plain batch cut: no operator gathers its input, gradients match eager."""
    torch.manual_seed(13)
    m, x = _ConvNet(), torch.randn(2, 3, 16, 16)
    procs = _procs(n)
    names = tuple(procs)
    sch = compile_module(m, (x,), procs, lambda nd: (dim, names, None) if nd.op == "placeholder" and nd.name == "x" else None, loss=0)
    assert not [st.target for st in sch.plan.steps if st.meta.get("fallback")]
    verbs = sch.structure["by_verb"]
    if dim == 0:
        assert set(verbs) == {"all_reduce"}
    else:
        assert verbs["halo"] == 2 and verbs["halo_back"] == 1              # the first layer's input needs no gradient
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


def _conv_rank(rank, world, rdv):
    torch.manual_seed(14)
    m, x = _ConvNet(), torch.randn(2, 3, 16, 16)
    procs = _procs(world)
    names = tuple(procs)
    sch = compile_module(m, (x,), procs, lambda nd: (2, names, None) if nd.op == "placeholder" and nd.name == "x" else None, loss=0)
    res = Program(sch)(x)                      # one process per processor: halos go point to point
    loss, grads = _eager(m, x)
    assert abs(float(res.outputs) - float(loss)) < 1e-5
    for k in ("c1.weight", "c2.weight", "fc.bias"):
        assert torch.allclose(res.parameters[k], grads[k], atol=1e-5), k


def test_halo_exchange_and_its_adjoint_between_processes():
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_conv_rank, 2, init_pg="gloo")


@pytest.mark.parametrize("dim", [0, 2])
def test_inference_batch_norm_keeps_batch_and_spatial_cuts(dim):
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c, self.bn = torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.BatchNorm2d(8)

        def forward(self, x):
            return torch.relu(self.bn(self.c(x)))

    torch.manual_seed(15)
    m = Net().eval()
    m.bn.running_mean.normal_()
    m.bn.running_var.uniform_(0.5, 2.0)
    x = torch.randn(4, 3, 8, 8)
    procs = _procs(2)
    names = tuple(procs)
    sch = compile_module(m, (x,), procs, lambda nd: (dim, names, None) if nd.op == "placeholder" and nd.name == "x" else None)
    assert sch.structure["fallbacks"] == 0 and sch.structure["by_verb"].get("all_gather") == 1      # only the result
    assert torch.allclose(Program(sch)(x), m(x), atol=1e-6)


def test_convolution_network_on_a_grid_batch_by_height():
    """A 2 x 2 grid: the batch over one axis, the image height over the other; halos travel along the second axis only."""
    torch.manual_seed(16)
    m, x = _ConvNet(), torch.randn(4, 3, 16, 16)
    procs = _procs(4)
    sch = compile_module(m, (x,), procs, lambda nd: ((0, 2), None, (None, None)) if nd.op == "placeholder" and nd.name == "x" else None,
                         loss=0, mesh=(2, 2))
    assert sch.structure["fallbacks"] == 0
    assert sch.structure["by_verb"]["halo"] == 2 and sch.structure["by_verb"]["halo_back"] == 1
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


def test_random_draws_do_not_depend_on_a_grid_cut():
    class Draws(torch.nn.Module):
        def forward(self, x):
            return torch.nn.functional.dropout(x, 0.5, training=True) + torch.rand_like(x)

    x = torch.ones(4, 8)
    grid = Program(compile_module(Draws(), (x,), _procs(4), lambda nd: ((0, 1), None, (None, None)) if nd.name == "x" else None, mesh=(2, 2)))(x)
    whole = Program(compile_module(Draws(), (x,), _procs(1), lambda nd: None))(x)
    assert torch.equal(grid, whole)


def test_recurrent_network_under_a_batch_cut():
    """An LSTM unrolls into splits, pointwise gates and joins: every piece keeps the batch cut, gradients are summed."""
    class Rnn(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.r, self.h = torch.nn.LSTM(8, 16, batch_first=True), torch.nn.Linear(16, 1)

        def forward(self, x):
            return self.h(self.r(x)[0]).pow(2).mean()

    torch.manual_seed(17)
    m, x = Rnn(), torch.randn(4, 5, 8)
    procs = _procs(2)
    sch = compile_module(m, (x,), procs, data_parallel(procs), loss=0)
    assert sch.structure["fallbacks"] == 0 and set(sch.structure["by_verb"]) == {"all_reduce"}
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


def test_constants_meet_partial_sums_only_after_the_reduction():
    """``sum over a cut dimension`` leaves partial sums; adding a constant, or dividing a constant by them, must wait
    for the reduction (each processor would otherwise apply the constant to its own partial)."""
    class Net(torch.nn.Module):
        def forward(self, x):
            s = x.sum(0)
            return s + 1.0, 2.0 - s, 3.0 / (s * s + 1.0), (s * 2.0) / 4.0, x.amax(0) * -1.0

    torch.manual_seed(18)
    x = torch.randn(6, 5)
    for n in (2, 3):
        procs = _procs(n)
        names = tuple(procs)
        out = Program(compile_module(Net(), (x,), procs, lambda nd: (0, names, None) if nd.name == "x" else None))(x)
        for got, ref in zip(out, Net()(x)):
            assert torch.allclose(got, ref, atol=1e-6)


def test_layers_on_different_processors_forward_and_backward():
    """A processor name per layer (a pipeline by placement): activations and their gradients go point to point, every
    gradient is reported from the processor that owns its layer."""
    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b, self.c = torch.nn.Linear(8, 16), torch.nn.Linear(16, 16), torch.nn.Linear(16, 4)

        def forward(self, x):
            return self.c(torch.relu(self.b(torch.relu(self.a(x))))).pow(2).mean()

    def placement(node):
        if node.op == "placeholder":
            if node.name == "x" or "p_a_" in node.name or "p_b_" in node.name:
                return "p0"
            return "p1" if "p_c_" in node.name else None
        quals = [q for _, (q, _) in (node.meta.get("nn_module_stack") or {}).items()]
        return "p1" if "c" in quals else "p0" if ("a" in quals or "b" in quals) else None

    torch.manual_seed(19)
    m, x = MLP(), torch.randn(6, 8)
    sch = compile_module(m, (x,), _procs(2), placement, loss=0)
    assert sch.structure["fallbacks"] == 0 and sch.structure["by_verb"]["send_recv"] >= 2
    assert "all_reduce" not in sch.structure["by_verb"] and "all_gather" not in sch.structure["by_verb"]
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)
    assert set(res.parameters) == set(grads) and all(g is not None for g in res.parameters.values())


@pytest.mark.parametrize("n", [3, 4])
def test_more_processors_than_samples_leaves_empty_shards(n):
    """A batch of 2 over 3 or 4 processors: the trailing shards are empty (the sizes of ``torch.chunk``), every operator,
    view and collective still runs, and the gradients are those of the whole batch."""
    torch.manual_seed(20)
    m = Decoder(dim=48, heads=4, ffn=96, layers=1)
    x = torch.randn(2, 6, 48)
    procs = _procs(n)
    sch = compile_module(m, (x,), procs, data_parallel(procs), loss=0)
    assert counts(2, None, n)[-1] == 0
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


@pytest.mark.parametrize("n", [2, 4])
def test_group_norm_under_a_batch_cut_takes_the_local_batch_size(n):
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c, self.gn = torch.nn.Conv2d(4, 8, 3, padding=1), torch.nn.GroupNorm(2, 8)

        def forward(self, x):
            return torch.relu(self.gn(self.c(x))).pow(2).mean()

    torch.manual_seed(21)
    m, x = Net(), torch.randn(6, 4, 8, 8)                                # 6 samples over 4 processors: 2, 2, 2, 0
    procs = _procs(n)
    sch = compile_module(m, (x,), procs, data_parallel(procs), loss=0)
    assert sch.structure["fallbacks"] == 0 and set(sch.structure["by_verb"]) == {"all_reduce"}
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


def test_sequence_parallel_megatron_layer_has_the_textbook_collectives():
    """Tokens and weights cut over the same processors: per layer one all-gather serves the query, key and value
    projections, one the two FFN input projections, and each row-parallel projection ends in a reduce-scatter; the
    activations (smaller than the weights here) are what is gathered.  All four become fused steps."""
    torch.manual_seed(22)
    m = Decoder(dim=512, heads=4, ffn=1024, layers=1).eval()
    x = torch.randn(1, 256, 512)
    procs = _procs(2)
    names = tuple(procs)
    tp = megatron(procs)
    sch = compile_module(m, (x,), procs, lambda nd: (1, names, None) if nd.op == "placeholder" and nd.name == "x" else tp(nd))
    assert sch.structure["by_verb"] == {"all_gather": 2, "reduce_scatter": 2, "all_reduce": 1}, sch.structure["by_verb"]
    prog = Program(sch)
    assert prog.fusion == {"ag_mm": 2, "mm_rs": 2, "rms_norm": 2, "ring_attention": 0}
    assert torch.allclose(prog(x), m(x), atol=1e-4)


def test_tensor_parallel_training_layer_needs_only_its_four_all_reduces():
    """Megatron tensor parallelism, forward and backward, batch of 2: the attention products keep batch and heads apart
    (so the cut along the heads survives them) and a layer costs two all-reduces forward and two backward.  The first
    layer's second backward all-reduce would only serve the gradient of its norm weight (the input needs none): that
    partial sum is scaled and summed over the rows first and goes out as one small all-reduce of the weight gradient.
    A partial sum with several readers is summed once and shared."""
    torch.manual_seed(23)
    procs = _procs(2)
    x = torch.randn(2, 12, 48)
    for layers in (1, 2):
        m = Decoder(dim=48, heads=4, ffn=96, layers=layers)
        sch = compile_module(m, (x,), procs, megatron(procs), loss=0)
        assert sch.structure["fallbacks"] == 0 and set(sch.structure["by_verb"]) == {"all_reduce"}
        big = [t for t in sch.plan.transfers if t.nbytes >= 2 * 12 * 48 * 4]
        assert len(big) == 4 * layers - 1, [(t.verb, t.nbytes) for t in sch.plan.transfers]
        assert len(sch.plan.transfers) == 4 * layers, [(t.verb, t.nbytes) for t in sch.plan.transfers]
    res = Program(sch)(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


def _bucket_rank(rank, world, rdv):
    torch.manual_seed(24)
    m = Decoder(dim=48, heads=4, ffn=96, layers=2)
    x = torch.randn(4, 12, 48)
    procs = _procs(world)
    prog = Program(compile_module(m, (x,), procs, data_parallel(procs), loss=0))
    assert prog.bucketed >= 18
    res = prog(x)
    loss, grads = _eager(m, x)
    _check(res, loss, grads)


def test_gradient_all_reduces_go_out_as_one_bucket(monkeypatch):
    """``MESH_BUCKET=1``: the all-reduces of gradients that nothing else reads are held back and reduced as one flat
    message per step, in the threaded interpreter and with one process per processor alike."""
    monkeypatch.setenv("MESH_BUCKET", "1")
    monkeypatch.setenv("MESH_SYNC_TRACE", "1")
    torch.manual_seed(24)
    m = Decoder(dim=48, heads=4, ffn=96, layers=2)
    x = torch.randn(4, 12, 48)
    procs = _procs(2)
    sch = compile_module(m, (x,), procs, data_parallel(procs), loss=0)
    prog = Program(sch)
    res = prog(x)
    assert prog.bucketed == sch.structure["by_verb"]["all_reduce"] - 1          # all but the loss
    assert len(prog.per_rank[0][0].trace) == 2                                    # the loss, then one bucket
    loss, grads = _eager(m, x)
    _check(res, loss, grads)
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_bucket_rank, 2, init_pg="gloo")


def test_invariant_values_are_recomputed_where_they_are_read():
    """A table that depends on no input, stated on one processor and read on another, is computed on both: no
    transfer carries it (duplicated cheap compute is free, a crossing is not)."""
    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = torch.nn.Linear(16, 16), torch.nn.Linear(16, 16)

        def forward(self, x):
            table = torch.sin(torch.arange(16, dtype=torch.float32) / 16.0) * 2.0
            return self.b(self.a(x) + table) * table
    torch.manual_seed(0)
    m = M().eval()
    x = torch.randn(4, 16)
    procs = {"p0": (0, "cpu"), "p1": (0, "cpu")}

    def placement(node):
        if node.name in ("arange", "div", "sin", "mul", "addmm", "add"):
            return "p0"
        if node.name in ("addmm_1", "mul_1"):
            return "p1"
        return None
    sch = compile_module(m, (x,), procs, placement)
    assert sch.structure["duplicated"] == 1
    moved = {t.value for t in sch.plan.transfers}
    assert not any(v.startswith(("mul", "sin", "arange", "div")) and not v.startswith("mul_1") for v in moved), moved
    out = Program(sch, threads=True)(x)
    assert torch.allclose(out, m(x), atol=1e-6)


def test_transfers_that_send_one_value_share_a_write():
    """Two transfers that publish the same value on one axis are one staged write with two members; an unrelated
    transfer is a write of its own; the structure report counts both."""
    from mesh_b200.compiler import schedule as S
    from mesh_b200.compiler.ir import Mesh, Plan, Ref, Step, Transfer

    def coll(verb, out, src, channel, kind):
        return Step("collective", out, verb, (Ref(src),), {}, {"axis": 0, "kind": kind, "to": None, "from": None, "channel": channel})
    steps = [Step("call", "h", "t", (Ref("x"),)),
             coll("all_gather", "h_all", "h", 0, "broadcast"),
             coll("broadcast", "h_b", "h", 1, "broadcast"),
             Step("call", "g", "u", (Ref("h_all"), Ref("h_b"))),
             coll("all_reduce", "g_sum", "g", 2, "reduce")]
    transfers = [Transfer(0, "broadcast", "all_gather", 0, "h", 0, (), nbytes=1024),
                 Transfer(1, "broadcast", "broadcast", 0, "h", 0, (), nbytes=1024),
                 Transfer(2, "reduce", "all_reduce", 0, "g", 0, (), nbytes=64)]
    plan = Plan(Mesh(("a", "b"), (2,)), steps, ["x"], {}, ["g_sum"], {}, transfers, {}, {})
    cp = S.copies(plan)
    assert len(cp.index) == 2
    assert sorted(map(sorted, cp.member.values())) == [[0, 1], [2]]
    assert cp.reusable == 1
    _, structure = S.schedule(plan)
    assert structure["writes"] == 2 and structure["shared_writes"] == 1


def test_pieces_of_a_concatenation_are_computed_in_place():
    """A rotary-style rotation (two pointwise halves, concatenated) under a batch cut: both halves have a destination,
    the concatenation runs without a copy (its result is the storage the halves were written into), and the numbers
    are those of eager execution; with the switch off nothing has a destination."""
    from mesh_b200.compiler import destine

    class Rotate(torch.nn.Module):
        def forward(self, x, c, s):
            a, b = x[..., :8], x[..., 8:]
            return torch.cat([a * c - b * s, b * c + a * s], -1) * 2.0

    torch.manual_seed(0)
    x, c, s = torch.randn(6, 4, 16), torch.randn(4, 8), torch.randn(4, 8)
    want = Rotate()(x, c, s)
    procs = _procs(2)

    def run(expect):
        sch = compile_module(Rotate(), (x, c, s), procs, data_parallel(procs))
        prog = Program(sch)
        got = prog(x, c, s)
        got = got[0] if isinstance(got, (tuple, list)) else got
        assert torch.allclose(got, want, atol=1e-6)
        execs = [r[0] for r in prog.per_rank if r is not None] if getattr(prog, "per_rank", None) else [prog.exec]
        assert all(e.destined == expect for e in execs)
        return sch

    sch = run(1)
    found = destine.analyse(sch.plan)
    assert len(found) == 2 and len({d.parent for d in found.values()}) == 1
    import os
    os.environ["MESH_DESTINED"] = "0"
    try:
        run(0)
    finally:
        del os.environ["MESH_DESTINED"]


def test_sequence_first_attention_keeps_a_batch_cut():
    """``nn.MultiheadAttention`` in its sequence-first layout ``[T, B, E]`` with the batch (the inner leading dimension)
    cut: the linear layers keep their leading dimensions apart, so the projections, the head split and the attention all
    run on the shard, and the only transfer is the gather of the result (the input itself is never gathered)."""
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.att = torch.nn.MultiheadAttention(32, 4, batch_first=False)

        def forward(self, x):
            return self.att(x, x, x, need_weights=False)[0]

    torch.manual_seed(0)
    m = Net().eval()
    x = torch.randn(6, 4, 32)
    procs = _procs(2)
    sch = compile_module(m, (x,), procs, lambda node: (1, tuple(procs), None) if node.op == "placeholder" and node.name == "x" else None)
    moved = [t.value for t in sch.plan.transfers]
    assert "x" not in moved and len(moved) == 1 and sch.structure["by_verb"] == {"all_gather": 1}
    assert any(st.target is torch.ops.aten.matmul.default for st in sch.plan.steps if st.op == "call")
    got = Program(sch)(x)
    got = got[0] if isinstance(got, (tuple, list)) else got
    assert torch.allclose(got, m(x), atol=1e-5)
    # a cut along the first dimension needs none of this and is captured as before
    sch0 = compile_module(m, (x,), procs, lambda node: (0, tuple(procs), None) if node.op == "placeholder" and node.name == "x" else None)
    assert not any(st.target is torch.ops.aten.matmul.default and len(sch0.plan.full_shapes[st.out]) == 3
                   for st in sch0.plan.steps if st.op == "call")
    got0 = Program(sch0)(x)
    got0 = got0[0] if isinstance(got0, (tuple, list)) else got0
    assert torch.allclose(got0, m(x), atol=1e-5)


def test_embedding_bag_keeps_a_column_cut_table():
    """A bag-of-embeddings table cut along the embedding dimension: the bags come out cut the same way, the layer that
    follows multiplies each processor's columns with the matching rows of its weight (the bias entering once), and the
    only transfer is the sum of those small partial products - neither the table nor the bags are gathered."""
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.bag = torch.nn.EmbeddingBag(50, 32, mode="sum")
            self.lin = torch.nn.Linear(32, 8)

        def forward(self, idx, off):
            return self.lin(self.bag(idx, off))

    torch.manual_seed(0)
    m = Net().eval()
    idx, off = torch.randint(0, 50, (20,)), torch.tensor([0, 3, 9, 15])
    procs = _procs(2)
    sch = compile_module(m, (idx, off), procs,
                         lambda node: (1, tuple(procs), None) if node.op == "placeholder" and node.name == "p_bag_weight" else None)
    assert sch.structure["fallbacks"] == 0
    assert [t.verb for t in sch.plan.transfers] == ["all_reduce"] and sch.structure["bytes_between_processors"] == 4 * 8 * 4
    got = Program(sch)(idx, off)
    got = got[0] if isinstance(got, (tuple, list)) else got
    assert torch.allclose(got, m(idx, off), atol=1e-6)


class _Blocks(torch.nn.Module):
    """The decoder's blocks without its loss: an inference graph, where attention stays one operator."""

    def __init__(self, layers=2):
        super().__init__()
        self.d = Decoder(dim=32, heads=4, ffn=64, layers=layers)

    def forward(self, x):
        for b in self.d.blocks:
            x = b(x)
        return x


@pytest.mark.parametrize("n,units", [(2, None), (3, (3, 1, 2)), (4, "striped"), (5, None)])
def test_context_parallel_attention_runs_as_a_ring(n, units, monkeypatch):
    """Tokens cut over the processors, contiguous, unequal, round-robin or with an empty share: the two gathers of keys
    and values in front of every attention become one ring step (blocks rotate, partial results merge by running
    maximum and sum, causal masks by positions in the whole sequence); what remains gathered is the output."""
    torch.manual_seed(31)
    m = _Blocks().eval()
    x = torch.randn(2, 12, 32)
    procs = _procs(n)
    sch = compile_module(m, (x,), procs, sequence_parallel(procs, units=units))
    assert sch.structure["by_verb"] == {"all_gather": 5} and sch.structure["gathering_fallbacks"] == 0
    prog = Program(sch)
    assert prog.fusion["ring_attention"] == 2
    rings = [st for st in prog.plan.steps if st.op == "fused" and st.target == "ring_attention"]
    assert len(rings) == 2 and all(st.meta["causal"] and st.meta["kind"] == "permute" for st in rings)
    assert sum(1 for st in prog.plan.steps if st.op == "collective") == 1
    ref = m(x)
    assert (prog(x) - ref).abs().max() <= 1e-5 * ref.abs().max()
    from mesh_b200.compiler import syncmon
    assert [v for v, *_ in syncmon.expected(prog.plan)].count("ring") == 2
    monkeypatch.setenv("MESH_RING_ATTENTION", "0")               # the gathered form computes the same numbers
    plain = Program(sch)
    assert plain.fusion.get("ring_attention", 0) == 0
    assert (plain(x) - ref).abs().max() <= 1e-5 * ref.abs().max()


def _ring_rank(rank, world, rdv):
    torch.manual_seed(32)
    m = _Blocks(layers=1).eval()
    x = torch.randn(2, 10, 32)
    procs = _procs(world)
    prog = Program(compile_module(m, (x,), procs, sequence_parallel(procs, units=(2, 1, 2))))
    assert prog.fusion["ring_attention"] == 1 and not prog.threads
    out = prog(x)                                                # blocks pass from process to process (point to point)
    if out is not None:
        ref = m(x)
        assert (out - ref).abs().max() <= 1e-5 * ref.abs().max()


def test_ring_attention_between_processes():
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_ring_rank, 3, init_pg="gloo")


def test_shared_tables_and_unused_parameters_in_training_graphs():
    """One table under three names of which the first is never read directly (encoder / decoder embeddings of a shared
    table), plus a head that this call does not use: the capture leaves out what gets no gradient, and the shared
    table's gradient - the sum over the names that are read - comes back under every one of its names."""
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.shared = torch.nn.Embedding(20, 8)
            self.enc = torch.nn.Embedding(20, 8)
            self.dec = torch.nn.Embedding(20, 8)
            self.enc.weight = self.shared.weight
            self.dec.weight = self.shared.weight
            self.mix = torch.nn.Linear(8, 8)
            self.unused = torch.nn.Linear(8, 3)

        def forward(self, a, b):
            return (self.mix(self.enc(a)) * self.dec(b)).sum(-1).pow(2).mean()

    torch.manual_seed(40)
    m = Net()
    a, b = torch.randint(0, 20, (4, 6)), torch.randint(0, 20, (4, 6))
    procs = _procs(2)
    names = tuple(procs)
    sch = compile_module(m, (a, b), procs, lambda n: (0, names, None) if n.op == "placeholder" and n.name in ("a", "b") else None, loss=0)
    assert sch.exported.tied == {"enc.weight": "shared.weight", "dec.weight": "shared.weight"}
    assert m.enc.weight is m.shared.weight and m.dec.weight is m.shared.weight and m.unused.weight.requires_grad
    res = Program(sch)(a, b)
    loss = m(a, b)
    loss.backward()
    assert abs(float(res.outputs.detach()) - float(loss.detach())) < 1e-5
    assert "unused.weight" not in res.parameters
    for name in ("shared.weight", "enc.weight", "dec.weight"):
        assert torch.allclose(res.parameters[name], m.shared.weight.grad, atol=1e-6), name
    assert torch.allclose(res.parameters["mix.weight"], m.mix.weight.grad, atol=1e-6)
