"""A zoo of ordinary torch modules, each compiled under a cut of its input along every kind of dimension (samples,
channels, space, features) and compared with eager PyTorch: outputs for inference graphs; loss, parameter gradients
(or input gradients, for modules without parameters) and buffer updates for training graphs.  Where the placement has a
rule that keeps the cut, the test also asserts that no operator had to gather an operand first."""
import copy

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from mesh_b200.compiler import Program, compile_module


def _procs(n):
    return {f"p{i}": (0, "cpu") for i in range(n)}


class _Loss(nn.Module):
    """A loss that no normalisation leaves invariant: a fixed pattern of weights plus the mean square."""

    def __init__(self, m):
        super().__init__()
        self.m = m

    def forward(self, x):
        y = self.m(x)
        y = y[0] if isinstance(y, (tuple, list)) else y
        w = torch.cos(torch.arange(y.numel(), dtype=torch.float32) * 0.37).view(y.shape)
        return (y.float() * w).mean() + (y.float() ** 2).mean()


class _Residual(nn.Module):
    def __init__(self):
        super().__init__()
        self.c1, self.b1 = nn.Conv2d(8, 8, 3, padding=1), nn.BatchNorm2d(8)
        self.c2, self.b2 = nn.Conv2d(8, 8, 3, padding=1), nn.BatchNorm2d(8)

    def forward(self, x):
        return F.relu(x + self.b2(self.c2(F.relu(self.b1(self.c1(x))))))


class _Pointwise(nn.Module):
    def forward(self, x):
        a = torch.softmax(x, -1) + torch.log_softmax(x, -1)
        b = torch.cumsum(x, 1) * x.sigmoid()
        c = torch.where(x > 0, x, torch.zeros_like(x)).clamp(-1, 1)
        d = x.mean(-1, keepdim=True) + x.var(-1, keepdim=True) + x.amax(-1, keepdim=True)
        return a + b + c + d + x.flip(1) + torch.roll(x, 1, 1) + F.elu(x) + torch.log1p(x.abs()) + torch.atan(x)


class _Extremes(nn.Module):
    def forward(self, x):
        v, i = x.topk(3, -1)
        s, _ = x.sort(-1)
        g = torch.gather(x, -1, i)
        return v.sum(-1) + g.sum(-1) + s[..., 0] + x.argmax(-1).float() + x.max(-1).values + x.min(-1)[0] + x.std(-1)


class _Padded(nn.Module):
    def forward(self, x):
        y = F.pad(x, (1, 1, 2, 0))
        return torch.cat([y, y * 2], 1)


class _Resized(nn.Module):
    def forward(self, x):
        return F.interpolate(x, scale_factor=2, mode="nearest") + F.interpolate(x, scale_factor=2, mode="bilinear", align_corners=False)


ZOO = {
    "strided_convolutions": (lambda: nn.Sequential(nn.Conv2d(3, 8, 3, stride=2, padding=1), nn.ReLU(), nn.Conv2d(8, 8, 3, padding=2, dilation=2)), (4, 3, 16, 16)),
    "patch_embedding": (lambda: nn.Sequential(nn.Conv2d(3, 8, 4, stride=4), nn.GELU()), (4, 3, 16, 16)),
    "learned_upsampling": (lambda: nn.Sequential(nn.ConvTranspose2d(4, 4, 2, stride=2), nn.ReLU()), (4, 4, 8, 8)),
    "depthwise_separable": (lambda: nn.Sequential(nn.Conv2d(8, 16, 3, padding=1, groups=8), nn.Conv2d(16, 8, 1)), (4, 8, 12, 12)),
    "residual_batch_norm": (_Residual, (4, 8, 12, 12)),
    "instance_norm": (lambda: nn.Sequential(nn.Conv2d(8, 8, 1), nn.InstanceNorm2d(8, affine=True)), (4, 8, 12, 12)),
    "group_norm": (lambda: nn.Sequential(nn.Conv2d(8, 8, 3, padding=1), nn.GroupNorm(2, 8), nn.SiLU()), (4, 8, 12, 12)),
    "volumes": (lambda: nn.Sequential(nn.Conv3d(2, 4, 3, padding=1), nn.MaxPool3d(2), nn.Conv3d(4, 4, 1), nn.AvgPool3d(2)), (4, 2, 8, 8, 8)),
    "pooled_classifier": (lambda: nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2), nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(8, 4)), (4, 3, 16, 16)),
    "activations": (lambda: nn.Sequential(nn.Linear(8, 8), nn.PReLU(), nn.Hardswish(), nn.ELU(), nn.LeakyReLU(), nn.Softplus(), nn.Mish(), nn.Hardtanh(), nn.ReLU6(), nn.LogSigmoid(), nn.CELU(), nn.SELU()), (4, 6, 8)),
    "pointwise_and_scans": (_Pointwise, (4, 6, 8)),
    "extremes": (_Extremes, (4, 6, 8)),
    "padded": (_Padded, (4, 6, 8)),
    "resized": (_Resized, (4, 3, 8, 8)),
    "encoder_layer": (lambda: nn.TransformerEncoderLayer(32, 4, 64, dropout=0.0, batch_first=True), (4, 6, 32)),
    "batch_norm_1d": (lambda: nn.Sequential(nn.Linear(8, 8), nn.BatchNorm1d(8)), (8, 8)),
}

# (model, cut dimension, training graph, the cut must survive every operator)
CASES = [
    ("strided_convolutions", 0, True, True), ("strided_convolutions", 1, True, True), ("strided_convolutions", 2, True, True),
    ("strided_convolutions", 3, False, True),
    ("patch_embedding", 2, True, True), ("patch_embedding", 1, False, True),
    ("learned_upsampling", 1, True, True), ("learned_upsampling", 2, True, True), ("learned_upsampling", 3, False, True),
    ("depthwise_separable", 1, True, True), ("depthwise_separable", 2, True, True),
    ("residual_batch_norm", 0, True, True), ("residual_batch_norm", 1, True, False), ("residual_batch_norm", 2, True, True),
    ("residual_batch_norm", 1, False, True),
    ("instance_norm", 0, True, True), ("instance_norm", 1, True, True), ("instance_norm", 3, True, True),
    ("group_norm", 0, True, True), ("group_norm", 2, False, False),
    ("volumes", 0, True, True), ("volumes", 1, True, True), ("volumes", 3, True, True),
    ("pooled_classifier", 0, True, True), ("pooled_classifier", 1, True, True), ("pooled_classifier", 2, True, True),
    ("activations", 0, True, True), ("activations", 1, False, True), ("activations", 2, True, True),
    ("pointwise_and_scans", 0, True, True), ("pointwise_and_scans", 1, True, False), ("pointwise_and_scans", 2, False, False),
    ("extremes", 0, True, True), ("extremes", 1, True, True), ("extremes", 2, False, False),
    ("padded", 0, True, True), ("padded", 1, False, False),
    ("resized", 0, True, True), ("resized", 1, True, True), ("resized", 2, False, False),
    ("encoder_layer", 0, True, True), ("encoder_layer", 1, True, True), ("encoder_layer", 2, False, False),
    ("batch_norm_1d", 0, True, True), ("batch_norm_1d", 1, True, True),
]


@pytest.mark.parametrize("name,dim,train,kept", CASES)
def test_module_under_a_cut_matches_eager(name, dim, train, kept):
    _run(name, dim, train, kept, 2, None)


# shares that are unequal, and shares that come out empty (more processors than channels or rows): operators that refuse
# empty operands are not called there; the executor states the empty or zero result itself
UNEVEN = [
    ("strided_convolutions", 1, True, 3, (3, 1, 2)), ("pooled_classifier", 1, True, 3, (3, 1, 2)),
    ("volumes", 1, True, 3, (3, 1, 2)), ("resized", 1, False, 3, (3, 1, 2)), ("residual_batch_norm", 1, True, 3, (1, 2, 1)),
    ("learned_upsampling", 2, True, 5, None), ("learned_upsampling", 1, True, 5, None), ("depthwise_separable", 1, True, 5, (4, 0, 1, 2, 1)),
    ("instance_norm", 0, True, 5, None), ("instance_norm", 2, True, 5, (5, 0, 3, 2, 2)), ("patch_embedding", 2, True, 5, None),
    ("extremes", 0, True, 5, None),
]


@pytest.mark.parametrize("name,dim,train,n,units", UNEVEN)
def test_module_under_uneven_and_empty_shares_matches_eager(name, dim, train, n, units):
    _run(name, dim, train, False, n, units)


def _run(name, dim, train, kept, n, units):
    make, shape = ZOO[name]
    torch.manual_seed(0)
    model = make()
    x = torch.randn(*shape)
    procs = _procs(n)
    names = tuple(procs)

    def place(node):
        val = node.meta.get("val")
        mine = node.op == "placeholder" and not node.name.startswith(("p_", "b_")) and getattr(val, "shape", None) == x.shape
        return (dim, names, units) if mine else None

    if not train:
        model.eval()
        sch = compile_module(model, (x,), procs, place)
        got, ref = Program(sch)(x), model(x)
        assert (got - ref).abs().max() <= 1e-5 * (ref.abs().max() + 1e-6)
    else:
        model = _Loss(model).train()
        bare = not list(model.parameters())
        if bare:
            x.requires_grad_(True)
        eager = copy.deepcopy(model)
        sch = compile_module(model, (x,), procs, place, loss=0)
        res = Program(sch)(x)
        ref = eager(x)
        ref.backward()
        assert abs(float(res.outputs.detach()) - float(ref.detach())) <= 1e-5 * max(1.0, abs(float(ref.detach())))
        if bare:
            wanted = {next(iter(res.inputs)): x.grad}
            given = res.inputs
        else:
            wanted = {k: p.grad for k, p in eager.named_parameters()}
            given = res.parameters
        scale = max(float(g.abs().max()) for g in wanted.values() if g is not None)
        for k, g in given.items():
            r = wanted[k]
            if r is None:
                continue
            if g.shape != r.shape:                           # a parameter that came back cut: this processor's block
                r = r[tuple(slice(0, n) for n in g.shape)]
            assert (g - r).abs().max() <= 2e-5 * scale, k
        for (k, a), (_, b) in zip(model.named_buffers(), eager.named_buffers()):
            assert (a.float() - b.float()).abs().max() <= 1e-5 * (b.float().abs().max() + 1e-6), k    # running statistics
    assert sch.signature.ok()
    if kept:
        assert sch.structure["gathering_fallbacks"] == 0, [str(s.target) for s in sch.plan.steps if s.meta.get("gathered")]


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("n", [2, 3])
def test_column_then_row_parallel_convolutions_need_one_all_reduce(transposed, n):
    """Output channels of the first convolution cut on its weight, input channels of the second cut to match: the pair
    runs with a single all-reduce of the second convolution's partial sums (the convolution form of a Megatron MLP)."""
    conv = nn.ConvTranspose2d if transposed else nn.Conv2d

    class Pair(nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = conv(4, 8, 3, padding=1), conv(8, 4, 3, padding=1)

        def forward(self, x):
            return self.b(F.relu(self.a(x)))

    torch.manual_seed(0)
    model = _Loss(Pair())
    x = torch.randn(2, 4, 8, 8)
    procs = _procs(n)
    names = tuple(procs)
    out_dim = 1 if transposed else 0
    stated = {"p_m_a_weight": out_dim, "p_m_a_bias": 0, "p_m_b_weight": 1 - out_dim}
    sch = compile_module(model, (x,), procs, lambda node: (stated[node.name], names, None) if node.name in stated else None, loss=0)
    assert sch.structure["by_verb"] == {"all_reduce": 1} and sch.structure["gathering_fallbacks"] == 0
    res = Program(sch)(x)
    ref = model(x)
    ref.backward()
    assert abs(float(res.outputs.detach()) - float(ref.detach())) < 1e-5
    scale = max(float(p.grad.abs().max()) for p in model.parameters())
    for k, g in res.parameters.items():
        r = dict(model.named_parameters())[k].grad
        if g.shape != r.shape:
            r = r[tuple(slice(0, m) for m in g.shape)]
        assert (g - r).abs().max() <= 2e-5 * scale, k


def _spd(x):
    return x @ x.mT + 4 * torch.eye(x.shape[-1])


# operators of the numerics table (transforms, complex numbers, distances, histograms, factorisations, scans, ranks,
# scatters, windows, samplers, norms, losses, contractions, repeats): a cut along the samples stays through all of them
NUMERICS = {
    "fourier": (lambda x: torch.fft.rfft(x, dim=-1).abs().sum(-1, keepdim=True) + torch.fft.fft(x, dim=-1).real
                + torch.fft.irfft(torch.fft.rfft(x, dim=-1), n=x.shape[-1], dim=-1), (4, 6, 16)),
    "fourier_2d": (lambda x: torch.fft.fft2(x).abs() + torch.fft.ifft2(torch.fft.fft2(x)).real, (4, 8, 8)),
    "complex": (lambda x: torch.view_as_real(torch.view_as_complex(x.reshape(4, 6, 8, 2))
                                             * torch.polar(torch.ones(8), torch.arange(8.) * 0.1)).flatten(-2), (4, 6, 16)),
    "distances": (lambda x: torch.cdist(x, x.flip(1)), (4, 6, 16)),
    "histogram": (lambda x: torch.histc(x, bins=8, min=-3, max=3), (4, 6, 16)),
    "determinant_inverse": (lambda x: torch.linalg.det(_spd(x))[..., None, None] * torch.linalg.inv(_spd(x)), (4, 6, 6)),
    "solves": (lambda x: torch.linalg.solve(_spd(x), x) + torch.cholesky_solve(x, torch.linalg.cholesky(_spd(x))), (4, 6, 6)),
    "spectra": (lambda x: torch.linalg.eigvalsh(_spd(x)) + torch.linalg.svdvals(x), (4, 6, 6)),
    "matrix_exponential": (lambda x: torch.linalg.matrix_exp(x * 0.1), (4, 6, 6)),
    "lu": (lambda x: torch.linalg.lu_factor(_spd(x))[0], (4, 6, 6)),
    "scans": (lambda x: x.cumsum(-1) + x.cumprod(-1) + x.cummax(-1).values + x.cummin(-1)[0] + torch.logcumsumexp(x, -1), (4, 6, 16)),
    "ranks": (lambda x: x.kthvalue(3, -1).values + x.median(-1).values + x.mode(-1).values + x.sort(-1).values[..., 0]
              + x.argsort(-1)[..., 0].float(), (4, 6, 16)),
    "scatters": (lambda x: torch.zeros(4, 6, 20).scatter_add(-1, (x.abs() * 5).long().clamp(0, 19), x)
                 + torch.zeros(4, 6, 20).index_add(-1, torch.arange(16), x), (4, 6, 16)),
    "windows": (lambda x: F.fold(F.unfold(x, 3, padding=1), (8, 8), 3, padding=1), (4, 2, 8, 8)),
    "sampler": (lambda x: F.grid_sample(x, torch.stack(torch.meshgrid(torch.linspace(-1, 1, 5), torch.linspace(-1, 1, 5),
                                                                      indexing="ij"), -1).expand(4, 5, 5, 2), align_corners=False), (4, 2, 8, 8)),
    "norms": (lambda x: F.layer_norm(x, (16,)) + F.normalize(x, dim=-1) + x.norm(dim=-1, keepdim=True)
              + torch.linalg.vector_norm(x, ord=1, dim=-1, keepdim=True) + F.rms_norm(x, (16,)), (4, 6, 16)),
    "losses": (lambda x: F.cross_entropy(x.flatten(0, 1), x.flatten(0, 1).argmax(-1), reduction="none").view(4, 6)
               + F.mse_loss(x, x.flip(-1), reduction="none").mean(-1)
               + F.kl_div(x.log_softmax(-1), x.flip(-1).softmax(-1), reduction="none").sum(-1)
               + F.binary_cross_entropy_with_logits(x, (x.flip(-1) > 0).float(), reduction="none").sum(-1), (4, 6, 16)),
    "contractions": (lambda x: torch.einsum("bij,bkj->bik", x, x).sum(-1) + torch.einsum("bij->bj", x)[:, :6]
                     + torch.einsum("bii->bi", x[..., :6]), (4, 6, 16)),
    "repeats": (lambda x: x.repeat(1, 2, 1)[:, :6] + x.repeat_interleave(2, dim=1)[:, :6] + x.tile((1, 1, 2))[..., :16], (4, 6, 16)),
    "blends": (lambda x: torch.lerp(x, x.flip(-1), 0.3) + torch.addcmul(x, x, x, value=0.5) + torch.addcdiv(x, x, x.abs() + 1)
               + torch.hypot(x, x.flip(-1)) + torch.atan2(x, x.flip(-1)) + x.frac() + torch.fmod(x, 2.0) + torch.remainder(x, 2.0), (4, 6, 16)),
    "pools_1d": (lambda x: F.avg_pool1d(x, 2).repeat(1, 1, 2) + F.max_pool1d(x, 2).repeat(1, 1, 2) + F.adaptive_avg_pool1d(x, 16), (4, 6, 16)),
}


class _Function(nn.Module):
    def __init__(self, f):
        super().__init__()
        self.f = f

    def forward(self, x):
        return self.f(x)


@pytest.mark.parametrize("name", sorted(NUMERICS))
def test_numerics_keep_a_cut_along_the_samples(name):
    f, shape = NUMERICS[name]
    torch.manual_seed(0)
    x = torch.randn(*shape)
    model = _Function(f).eval()
    procs = _procs(2)
    names = tuple(procs)
    sch = compile_module(model, (x,), procs, lambda node: (0, names, None) if node.op == "placeholder" and node.name == "x" else None)
    got, ref = Program(sch)(x), model(x)
    assert (got - ref).abs().max() <= 1e-5 * (ref.abs().max() + 1e-6)
    assert sch.structure["gathering_fallbacks"] == 0, [str(s.target) for s in sch.plan.steps if s.meta.get("gathered")]
    if name == "histogram":                                    # every processor counts its own elements: one small sum
        assert sch.structure["by_verb"] == {"all_reduce": 1}


def _zoo_rank(rank, world, rdv):
    # channel-parallel, strided-halo and depthwise convolutions with norms, one process per processor
    for name, dim in (("strided_convolutions", 1), ("strided_convolutions", 2), ("depthwise_separable", 1), ("residual_batch_norm", 0)):
        make, shape = ZOO[name]
        torch.manual_seed(0)
        model = _Loss(make()).train()
        eager = copy.deepcopy(model)
        x = torch.randn(*shape)
        procs = _procs(world)
        names = tuple(procs)

        def place(node):
            val = node.meta.get("val")
            mine = node.op == "placeholder" and not node.name.startswith(("p_", "b_")) and getattr(val, "shape", None) == x.shape
            return (dim, names, None) if mine else None
        prog = Program(compile_module(model, (x,), procs, place, loss=0))
        assert not prog.threads
        res = prog(x)
        ref = eager(x)
        ref.backward()
        assert abs(float(res.outputs.detach()) - float(ref.detach())) <= 1e-5 * max(1.0, abs(float(ref.detach()))), name
        scale = max(float(p.grad.abs().max()) for p in eager.parameters())
        for k, g in res.parameters.items():
            r = dict(eager.named_parameters())[k].grad
            if g is not None and g.shape == r.shape:
                assert (g - r).abs().max() <= 2e-5 * scale, (name, k)


def test_zoo_models_between_processes():
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_zoo_rank, 2, init_pg="gloo")


# the same functions differentiated: the backward operators keep the cut too (input gradients against eager's)
DIFFERENTIATED = ["fourier_2d", "complex", "distances", "determinant_inverse", "solves", "spectra", "matrix_exponential", "lu",
                  "scans", "scatters", "windows", "sampler", "norms", "losses", "contractions", "repeats", "blends", "pools_1d"]


@pytest.mark.parametrize("name", DIFFERENTIATED)
def test_numerics_backward_keeps_a_cut_along_the_samples(name):
    f, shape = NUMERICS[name]
    torch.manual_seed(0)
    x = torch.randn(*shape, requires_grad=True)
    model = _Loss(_Function(f))
    procs = _procs(2)
    names = tuple(procs)
    sch = compile_module(model, (x,), procs, lambda node: (0, names, None) if node.op == "placeholder" and node.name == "x" else None, loss=0)
    res = Program(sch)(x)
    ref = model(x)
    ref.backward()
    assert abs(float(res.outputs.detach()) - float(ref.detach())) <= 1e-5 * max(1.0, abs(float(ref.detach())))
    got = next(iter(res.inputs.values()))
    want = x.grad[: got.shape[0]] if got.shape != x.grad.shape else x.grad
    assert (got - want).abs().max() <= 2e-4 * (want.abs().max() + 1e-9)
    assert sch.structure["gathering_fallbacks"] == 0, [str(s.target) for s in sch.plan.steps if s.meta.get("gathered")]
