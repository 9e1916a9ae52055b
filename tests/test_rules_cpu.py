"""Many small operator graphs under several cuts: whatever the rules decide, results equal the unsharded module."""
import pytest
import torch

from mesh_b200.compiler import Program, compile_module

F = torch.nn.functional
CASES = {
 "softmax_cut_dim": lambda x: torch.softmax(x, 0),
 "logsumexp": lambda x: torch.logsumexp(x, 0) + torch.logsumexp(x, 1).sum(),
 "max_vals": lambda x: x.max(0).values + x.min(1).values.sum(),
 "argmax": lambda x: x.argmax(0).float() + x.argmax(1).float().sum(),
 "cumsum": lambda x: x.cumsum(0) + x.cumsum(1),
 "var": lambda x: x.var(0) + x.std(1).sum(),
 "norm": lambda x: x.norm(dim=0) + x.norm(),
 "mean_mul": lambda x: x.mean(0) * x.mean(1).sum() + x.mean(),
 "prod": lambda x: (x * 0.1 + 1).prod(0),
 "matmul_t": lambda x: x.T @ x + (x @ x.T).sum(),
 "where": lambda x: torch.where(x > 0, x, x * 0.1).sum(0) + 1,
 "clamp_sum": lambda x: x.clamp(min=0).sum(0).sqrt() + 1e-3,
 "amax_neg": lambda x: -x.amax(0) + (x.amax(0) + 1) * 2,
 "sort": lambda x: x.sort(0).values + x.sort(1).values,
 "topk": lambda x: x.topk(2, 0).values.sum(0) + x.topk(2, 1).values.sum(1).sum(),
 "flip_roll": lambda x: x.flip(0) + x.roll(1, 0) + x.flip(1),
 "pad": lambda x: F.pad(x, (1, 1, 2, 0)).sum(0),
 "index": lambda x: x[torch.tensor([0, 2, 1])].sum(0) + x[:, torch.tensor([1, 0])].sum(),
 "expand_bcast": lambda x: (x[:, None, :] * x[None, :, :]).sum((0, 2)),
 "layer_norm": lambda x: F.layer_norm(x, (x.shape[1],)) + F.layer_norm(x.T, (x.shape[0],)).T,
 "einsum": lambda x: torch.einsum("ij,kj->ik", x, x).sum(1) + torch.einsum("ij,ik->jk", x, x).sum(),
 "div_const": lambda x: 1.0 / (x.sum(0).abs() + 1) + (x.sum(0) / 3),
 "any_all": lambda x: (x > 0).any(0).float() + (x > -5).all(0).float(),
 "mse": lambda x: F.mse_loss(x, x.flip(0)) + F.l1_loss(x, torch.zeros_like(x)),
 "tril": lambda x: torch.tril(x @ x.T).sum(0),
 "gather": lambda x: x.gather(1, x.argsort(1)) .sum(0) + x.gather(0, x.argsort(0)).sum(),
 "repeat": lambda x: x.repeat(2, 1).sum(0) + x.repeat_interleave(2, 0).sum(0),
 "stack_cat": lambda x: torch.stack([x, x * 2]).sum((0, 1)) + torch.cat([x, x], 0).sum(0) + torch.cat([x, x], 1).sum(),
 "count": lambda x: (x > 0).sum(0).float() / x.shape[0] + (x > 0).float().mean(),
}

CUTS = [(2, 1, None), (3, 0, "striped"), (2, 0, (2, 1))]


@pytest.mark.parametrize("name", sorted(CASES))
def test_operator_graph_matches_eager_under_every_cut(name):
    fn = CASES[name]

    class Net(torch.nn.Module):
        def forward(self, x):
            return fn(x)

    torch.manual_seed(0)
    x = torch.randn(6, 4)
    ref = fn(x)
    for n, dim, units in CUTS:
        procs = {f"p{i}": (0, "cpu") for i in range(n)}
        names = tuple(procs)
        sch = compile_module(Net(), (x,), procs, lambda nd: (dim, names, units) if nd.name == "x" else None)
        out = Program(sch)(x)
        assert out.shape == ref.shape, (n, dim, units)
        assert torch.allclose(out.float(), ref.float(), atol=1e-4), (n, dim, units, sch.structure["fallbacks"])


# ---- training graphs: fn(x [6, 4], w [4, 5], v [5]) -> loss; the data and / or the weight are cut
TRAINING = {
 "linear_relu": lambda x, w, v: (torch.relu(x @ w) * v).sum(),
 "softmax_ce": lambda x, w, v: F.cross_entropy((x @ w) * v, torch.arange(6) % 5),
 "mean_var": lambda x, w, v: ((x @ w).var(0) * v).sum() + (x @ w).mean(),
 "norm_rows": lambda x, w, v: F.normalize(x @ w, dim=1).mul(v).sum(),
 "norm_cols": lambda x, w, v: F.normalize(x @ w, dim=0).mul(v).sum(),
 "max_pool_rows": lambda x, w, v: (x @ w).max(0).values.dot(v),
 "logsumexp0": lambda x, w, v: torch.logsumexp(x @ w, 0).dot(v),
 "layernorm": lambda x, w, v: F.layer_norm(x @ w, (5,), v, v * 0.5).pow(2).mean(),
 "gelu_dropout0": lambda x, w, v: F.dropout(F.gelu(x @ w), 0.0).sum() + v.sum(),
 "bilinear": lambda x, w, v: ((x @ w) * (x @ w).flip(0)).sum() * v.mean(),
 "tanh_chain": lambda x, w, v: torch.tanh(torch.tanh(x @ w) @ w.T @ w).mean() + (v * v).sum(),
 "cumsum_rows": lambda x, w, v: (x @ w).cumsum(0).mul(v).mean(),
 "weight_norm": lambda x, w, v: (x @ (w / w.norm(dim=0, keepdim=True))).pow(2).sum() + v.norm(),
 "embedding": lambda x, w, v: F.embedding(torch.arange(6) % 4, w).mul(v).sum() + (x * 0).sum(),
 "mse_target": lambda x, w, v: F.mse_loss(x @ w, torch.ones(6, 5)) + F.smooth_l1_loss((x @ w) * v, torch.zeros(6, 5)),
 "outer": lambda x, w, v: torch.einsum("bi,bj->ij", x, x @ w).mul(w).sum() + v.sum(),
 "where_mask": lambda x, w, v: torch.where((x @ w) > 0, x @ w, 0.1 * (x @ w)).mul(v).mean(),
 "sort_vals": lambda x, w, v: (x @ w).sort(0).values[-2:].mul(v).sum(),
 "exp_sum_div": lambda x, w, v: ((x @ w).exp() / ((x @ w).exp().sum(0) + 1.0)).mul(v).sum(),
}

TRAINING_CUTS = [(3, (0, "striped"), None), (2, None, (1, None)), (2, (0, None), (1, None)), (2, (1, None), (0, None))]


@pytest.mark.parametrize("name", sorted(TRAINING))
def test_training_graph_loss_and_gradients_match_eager_under_every_cut(name):
    fn = TRAINING[name]

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            g = torch.Generator().manual_seed(1)
            self.w = torch.nn.Parameter(torch.randn(4, 5, generator=g))
            self.v = torch.nn.Parameter(torch.randn(5, generator=g))

        def forward(self, x):
            return fn(x, self.w, self.v)

    torch.manual_seed(0)
    x = torch.randn(6, 4)
    ref = Net()
    loss = ref(x)
    loss.backward()
    for n, xcut, wcut in TRAINING_CUTS:
        procs = {f"p{i}": (0, "cpu") for i in range(n)}
        names = tuple(procs)

        def placement(nd):
            if nd.op != "placeholder":
                return None
            if nd.name == "x" and xcut:
                return (xcut[0], names, xcut[1])
            if nd.name == "p_w" and wcut:
                return (wcut[0], names, wcut[1])
            return None
        res = Program(compile_module(Net(), (x,), procs, placement, loss=0), threads=True)(x)
        assert abs(float(res.outputs) - float(loss)) < 1e-4, (n, xcut, wcut)
        gw = res.parameters["w"]
        want = ref.w.grad if gw.shape == ref.w.grad.shape else ref.w.grad.narrow(wcut[0], 0, gw.shape[wcut[0]])   # processor 0's shard
        assert torch.allclose(gw, want, atol=1e-4), (n, xcut, wcut)
        assert torch.allclose(res.parameters["v"], ref.v.grad, atol=1e-4), (n, xcut, wcut)


def _dist_rank(rank, world, rdv):
    """One process per processor (gloo): unequal cuts, which need per-rank counts in every collective."""
    torch.manual_seed(0)
    x = torch.randn(6, 4)
    procs = {f"p{i}": (0, "cpu") for i in range(world)}
    names = tuple(procs)
    for name, fn in CASES.items():
        class Net(torch.nn.Module):
            def forward(self, x):
                return fn(x)
        out = Program(compile_module(Net(), (x,), procs, lambda nd: (0, names, (2, 1)) if nd.name == "x" else None))(x)
        if out is not None:
            assert torch.allclose(out.float(), fn(x).float(), atol=1e-4), name
    for name in ("linear_relu", "layernorm", "sort_vals", "exp_sum_div", "outer"):
        fn = TRAINING[name]

        class Train(torch.nn.Module):
            def __init__(self):
                super().__init__()
                g = torch.Generator().manual_seed(1)
                self.w = torch.nn.Parameter(torch.randn(4, 5, generator=g))
                self.v = torch.nn.Parameter(torch.randn(5, generator=g))

            def forward(self, x):
                return fn(x, self.w, self.v)
        ref = Train()
        loss = ref(x)
        loss.backward()
        for xcut, wcut in (((0, None), (1, None)), (None, (1, None))):           # the weight's 5 columns: 3 + 2

            def placement(nd):
                if nd.op != "placeholder":
                    return None
                if nd.name == "x" and xcut:
                    return (xcut[0], names, xcut[1])
                return (wcut[0], names, wcut[1]) if nd.name == "p_w" else None
            res = Program(compile_module(Train(), (x,), procs, placement, loss=0))(x)
            assert abs(float(res.outputs) - float(loss)) < 1e-4, name
            gw = res.parameters["w"]
            start = 0 if rank == 0 else 3
            assert torch.allclose(gw, ref.w.grad[:, start:start + gw.shape[1]], atol=1e-4), name
            assert torch.allclose(res.parameters["v"], ref.v.grad, atol=1e-4), name


def test_one_process_per_processor_with_unequal_cuts():
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_dist_rank, 2, init_pg="gloo", timeout=900)


GRIDS = [((0, None), (None, 1)), ((0, 1), (None, None))]      # (cut of x, cut of w) per grid axis


@pytest.mark.parametrize("name", sorted(TRAINING))
def test_training_graph_on_a_two_by_two_grid(name):
    fn = TRAINING[name]

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            g = torch.Generator().manual_seed(1)
            self.w = torch.nn.Parameter(torch.randn(4, 5, generator=g))
            self.v = torch.nn.Parameter(torch.randn(5, generator=g))

        def forward(self, x):
            return fn(x, self.w, self.v)

    torch.manual_seed(0)
    x = torch.randn(6, 4)
    ref = Net()
    loss = ref(x)
    loss.backward()
    procs = {f"p{i}": (0, "cpu") for i in range(4)}
    for xd, wd in GRIDS:
        def placement(nd):
            if nd.op != "placeholder":
                return None
            if nd.name == "x" and any(d is not None for d in xd):
                return (xd, None, (None, None))
            if nd.name == "p_w" and any(d is not None for d in wd):
                return (wd, None, (None, None))
            return None
        res = Program(compile_module(Net(), (x,), procs, placement, loss=0, mesh=(2, 2)), threads=True)(x)
        assert abs(float(res.outputs) - float(loss)) < 1e-4, (xd, wd)
        assert torch.allclose(res.parameters["v"], ref.v.grad, atol=1e-4), (xd, wd)
        gw, want = res.parameters["w"], ref.w.grad
        for d in range(2):                                       # processor 0 holds the first block of a cut weight
            if gw.shape[d] != want.shape[d]:
                want = want.narrow(d, 0, gw.shape[d])
        assert torch.allclose(gw, want, atol=1e-4), (xd, wd)


# ---- views and batched products of a [4, 6, 8] tensor
VIEWS = {
 "merge01": lambda x: x.reshape(24, 8).sum(0),
 "merge12": lambda x: x.reshape(4, 48).sum(1),
 "split2": lambda x: x.reshape(4, 6, 2, 4).sum((1, 3)),
 "split0": lambda x: x.reshape(2, 2, 6, 8).sum((0, 2)),
 "split1": lambda x: x.reshape(4, 3, 2, 8).sum((2,)),
 "flatten_all": lambda x: x.reshape(-1).cumsum(0)[-1:],
 "transpose_merge": lambda x: x.transpose(0, 1).reshape(6, 32).sum(1),
 "permute_merge": lambda x: x.permute(2, 0, 1).reshape(8, 24) @ torch.ones(24, 3),
 "heads": lambda x: x.reshape(4, 6, 2, 4).transpose(1, 2).reshape(8, 6, 4).sum((1, 2)),
 "bmm": lambda x: torch.bmm(x, x.transpose(1, 2)).sum((1, 2)),
 "bmm_merge": lambda x: torch.bmm(x, x.transpose(1, 2)).reshape(24, 6).sum(1),
 "unsqueeze_expand": lambda x: x.unsqueeze(1).expand(4, 3, 6, 8).reshape(12, 48).sum(1),
 "squeeze": lambda x: x[:, :1].squeeze(1) + x.sum(1),
 "select": lambda x: x[:, 2] + x[1].sum(0) + x[..., 3].sum(),
 "narrow": lambda x: x[:, 1:4].sum(1) + x[1:3].sum((0, 1)) ,
 "chunk": lambda x: sum(c.sum(1) for c in x.chunk(3, 1)) + sum(c.sum() for c in x.chunk(2, 0)),
 "unfold_like": lambda x: x.reshape(4, 2, 3, 8)[:, :, 1:].reshape(4, 4, 8).sum(1),
 "movedim": lambda x: x.movedim(0, 2).contiguous().view(48, 4).sum(0),
 "linear3d": lambda x: torch.nn.functional.linear(x, torch.ones(5, 8)).sum(1),
 "mean_dims": lambda x: x.mean((0, 2)) + x.mean(1).sum(),
 "softmax3d": lambda x: torch.softmax(x, 1).sum(2).sum(1) + torch.softmax(x, 2).sum(1).sum(1) + torch.softmax(x, 0).sum((1, 2)),
}

VIEW_CUTS = [(2, 0, None), (3, 1, "striped"), (2, 2, (1, 2))]


@pytest.mark.parametrize("name", sorted(VIEWS))
def test_views_of_a_cut_tensor_match_eager(name):
    fn = VIEWS[name]

    class Net(torch.nn.Module):
        def forward(self, x):
            return fn(x)

    torch.manual_seed(0)
    x = torch.randn(4, 6, 8)
    ref = fn(x)
    for n, dim, units in VIEW_CUTS:
        procs = {f"p{i}": (0, "cpu") for i in range(n)}
        names = tuple(procs)
        out = Program(compile_module(Net(), (x,), procs, lambda nd: (dim, names, units) if nd.name == "x" else None))(x)
        assert out.shape == ref.shape and torch.allclose(out, ref, atol=1e-4), (n, dim, units)


@pytest.mark.parametrize("causal", [False, True])
def test_whole_attention_under_every_cut(causal):
    """Inference graphs keep attention as one operator: heads or batch cut -> local; queries cut along the sequence ->
    local when not causal; anything else gathers.  Every combination equals the unsharded result."""
    class Attn(torch.nn.Module):
        def forward(self, q, k, v):
            return F.scaled_dot_product_attention(q, k, v, is_causal=causal)

    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 4, 6, 8) for _ in range(3))
    ref = Attn()(q, k, v)
    for n, dim, units in ((2, 0, None), (2, 1, None), (2, 2, None), (3, 2, "striped"), (2, 3, None)):
        procs = {f"p{i}": (0, "cpu") for i in range(n)}
        names = tuple(procs)
        for which in (("q", "k", "v"), ("q",), ("k", "v")):
            sch = compile_module(Attn(), (q, k, v), procs, lambda nd: (dim, names, units) if nd.name in which else None)
            assert torch.allclose(Program(sch)(q, k, v), ref, atol=1e-5), (n, dim, units, which)
            if dim in (0, 1) and which == ("q", "k", "v"):
                assert sch.structure["by_verb"] == {"all_gather": 1}          # only the result is brought together
            if dim == 2 and which == ("q", "k", "v"):
                # queries stay cut (with their rows of the causal mask); keys, values and the result are gathered
                assert sch.structure["fallbacks"] == 0 and sch.structure["by_verb"] == {"all_gather": 3}


def test_one_dimension_cut_along_two_grid_axes_is_refused_with_a_reason():
    import pytest
    from mesh_b200.compiler import compile_module
    m = torch.nn.Linear(8, 8)
    x = torch.randn(4, 8)
    procs = {f"p{i}": (0, "cpu") for i in range(4)}
    with pytest.raises(ValueError, match="more than one axis"):
        compile_module(m, (x,), procs, lambda n: ((0, 0), None, (None, None)) if n.name == "input" or n.name == "x" else None, mesh=(2, 2))
