"""tcgen05 GEMM and its fused epilogues against a plain PyTorch fp32 statement of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(got, want, tol=4e-3):
    from _oracle import assert_close_rms
    assert_close_rms(got, want, tol=tol)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 768, 512), (200, 264, 328), (4096, 1024, 1024)])
def test_gemm_kmajor(M, N, K):
    from mesh_b200.ops.gemm import gemm
    from mesh_b200.utils.status import check_status
    a, b = _rand((M, K), seed=1), _rand((N, K), seed=2)
    out = gemm(a, b)
    check_status()
    _close(out, a.float() @ b.float().T)


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 320), (448, 832, 1000)])
def test_gemm_mn_major(a_mn, b_mn, M, N, K):
    from mesh_b200.ops.gemm import gemm
    from mesh_b200.utils.status import check_status
    a = _rand((K, M) if a_mn else (M, K), seed=3)
    b = _rand((K, N) if b_mn else (N, K), seed=4)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    check_status()
    af = a.float().T if a_mn else a.float()
    bf = b.float().T if b_mn else b.float()
    _close(out, af @ bf.T)


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("M,F,K", [(128, 128, 64), (256, 384, 256), (300, 608, 512)])
def test_glu_fwd(act, M, F, K):
    from mesh_b200.ops.gemm import glu_fwd
    from mesh_b200.utils.status import check_status
    x, w = _rand((M, K), seed=5), _rand((2 * F, K), 0.05, seed=6)
    h, gu = glu_fwd(x, w, act=act)
    check_status()
    g = x.float() @ w[:F].float().T
    u = x.float() @ w[F:].float().T
    a = torch.nn.functional.silu(g) if act == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
    _close(gu[:, :F], g)
    _close(gu[:, F:], u)
    _close(h, a * u, 6e-3)


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("M,F,D", [(128, 256, 64), (256, 512, 256), (300, 576, 384)])
def test_glu_bwd(act, M, F, D):
    from mesh_b200.ops.gemm import glu_bwd
    from mesh_b200.utils.status import check_status
    dy, wd, gu = _rand((M, D), seed=7), _rand((D, F), 0.05, seed=8), _rand((M, 2 * F), seed=9)
    out = glu_bwd(dy, wd, gu, act=act)
    check_status()
    g = gu[:, :F].float().requires_grad_(True)
    u = gu[:, F:].float().requires_grad_(True)
    a = torch.nn.functional.silu(g) if act == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
    dh = dy.float() @ wd.float()
    (a * u).backward(dh)
    _close(out[:, :F], g.grad, 6e-3)
    _close(out[:, F:], u.grad, 6e-3)


@pytest.mark.parametrize("M,D,F", [(512, 256, 640), (2048, 1024, 4096), (384, 512, 1152)])
def test_glu_ffn_autograd(M, D, F):
    """The second shape has several waves of tiles per launch, so the chained launches of a pass (dependent launches
    gated by row-block counters) really overlap; the third has an odd number of row blocks."""
    from mesh_b200.ops.gemm import glu_ffn
    from mesh_b200.utils.status import check_status
    x = _rand((M, D), seed=10).requires_grad_(True)
    wgu = _rand((2 * F, D), 0.05, seed=11).requires_grad_(True)
    wd = _rand((D, F), 0.05, seed=12).requires_grad_(True)
    y = glu_ffn(x, wgu, wd)
    dy = _rand((M, D), seed=13)
    y.backward(dy)
    check_status()
    xr, wgur, wdr = (t.detach().float().requires_grad_(True) for t in (x, wgu, wd))
    g = xr @ wgur[:F].T
    u = xr @ wgur[F:].T
    yr = (torch.nn.functional.silu(g) * u) @ wdr.T
    yr.backward(dy.float())
    _close(y, yr, 8e-3)
    _close(x.grad, xr.grad, 8e-3)
    _close(wgu.grad, wgur.grad, 8e-3)
    _close(wd.grad, wdr.grad, 8e-3)


def test_chained_launches_give_the_same_bits_as_serial_ones(monkeypatch):
    from mesh_b200.ops.gemm import glu_ffn
    from mesh_b200.utils.status import check_status
    M, D, F = 2048, 1024, 4096
    outs = []
    for mode in ("1", "0", "1"):
        monkeypatch.setenv("MESH_GEMM_CHAIN", mode)
        x = _rand((M, D), seed=10).requires_grad_(True)
        wgu = _rand((2 * F, D), 0.05, seed=11).requires_grad_(True)
        wd = _rand((D, F), 0.05, seed=12).requires_grad_(True)
        for _ in range(3):
            x.grad = wgu.grad = wd.grad = None
            y = glu_ffn(x, wgu, wd)
            y.backward(_rand((M, D), seed=13))
        check_status()
        outs.append((y.detach(), x.grad, wgu.grad, wd.grad))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    for a, b in zip(outs[0], outs[2]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (384, 1000, 2048), (4096, 2048, 2048), (200, 264, 320)])
def test_gemm_with_group_quantised_weights(bits, M, N, K):
    """Codes dequantised in registers by the GEMM's producer warps, against the dequantised matrix in fp32."""
    from mesh_b200.ops.decode import dequantize_w4, dequantize_w8, quantize_w4, quantize_w8
    from mesh_b200.ops.gemm import gemm_q
    from mesh_b200.utils.status import check_status
    a = _rand((M, K), seed=21)
    w = _rand((N, K), 0.05, seed=22)
    codes, scales = (quantize_w4 if bits == 4 else quantize_w8)(w)
    wd = (dequantize_w4 if bits == 4 else dequantize_w8)(codes, scales)
    for pair, tile_n in ((0, 0), (-1, 256), (0, 128), (-1, 128)):
        out = gemm_q(a, codes, scales, pair=pair, tile_n=tile_n)
        check_status()
        _close(out, a.float() @ wd.float().T)


def test_coded_linear_uses_the_kernels_for_any_batch():
    from mesh_b200.ops.fragment import CodedLinear
    w = _rand((1024, 2048), 0.05, seed=23)
    for bits in (4, 8):
        lin = CodedLinear(w, bits=bits).cuda()
        for rows in (3, 8, 9, 700):
            x = _rand((rows, 2048), seed=24 + rows)
            _close(lin(x), x.float() @ lin.dense().float().T)
