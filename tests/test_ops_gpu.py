"""RMSNorm, RoPE and router top-k kernels against fp32 PyTorch statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 2048), (7, 1536), (300, 4096), (64, 8192)])
def test_rmsnorm_fwd(rows, cols):
    from mesh_b200.ops.norm import rmsnorm_fwd, rmsnorm_ref
    x = torch.randn(rows, cols, device="cuda").bfloat16()
    w = (torch.randn(cols, device="cuda") * 0.1 + 1).bfloat16()
    y, _, _ = rmsnorm_fwd(x, w, 1e-6)
    torch.testing.assert_close(y.float(), rmsnorm_ref(x, w).float(), atol=2e-2, rtol=2e-2)
    r = torch.randn(rows, cols, device="cuda").bfloat16()
    y2, res, _ = rmsnorm_fwd(x, w, 1e-6, residual=r, weight_offset=1.0)
    s = (x.float() + r.float()).bfloat16()
    torch.testing.assert_close(res.float(), s.float(), atol=1e-2, rtol=1e-2)
    torch.testing.assert_close(y2.float(), rmsnorm_ref(s, w, weight_offset=1.0).float(), atol=3e-2, rtol=3e-2)


def test_rmsnorm_bwd():
    from mesh_b200.ops.norm import rmsnorm
    x = torch.randn(500, 2048, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(2048, device="cuda") * 0.1 + 1).bfloat16().requires_grad_(True)
    dy = torch.randn(500, 2048, device="cuda").bfloat16()
    rmsnorm(x, w).backward(dy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    yr.backward(dy.float())
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, atol=0.5, rtol=3e-2)


@pytest.mark.parametrize("heads,hd", [(8, 256), (16, 128), (2, 64)])
def test_rope(heads, hd):
    from mesh_b200.ops.rope import rope_, rope_ref, rope_tables
    T = 77
    cos, sin = rope_tables(1024, hd, theta=1e6)
    pos = torch.randint(0, 1024, (T,), device="cuda", dtype=torch.int32)
    x = torch.randn(T, heads, hd, device="cuda").bfloat16()
    want = rope_ref(x, pos, cos, sin)
    got = rope_(x.clone(), pos, cos, sin)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    back = rope_(got.clone(), pos, cos, sin, inverse=True)
    torch.testing.assert_close(back.float(), x.float(), atol=4e-2, rtol=4e-2)


@pytest.mark.parametrize("E,k", [(64, 6), (8, 2), (256, 8), (40, 3)])
def test_router_topk(E, k):
    from mesh_b200.ops.router import router_topk, router_topk_ref
    T = 1000
    logits = torch.randn(T, E, device="cuda")
    bias = torch.randn(E, device="cuda")
    w, i = router_topk(logits, k, bias)
    wr, ir = router_topk_ref(logits, k, bias)
    assert torch.equal(i, ir)
    torch.testing.assert_close(w, wr, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("n", [8, 1000, 4096 * 512, 4096 * 4096 + 3])
def test_dot_sum(n):
    from mesh_b200.ops.loss import dot_sum
    a = torch.randn(n, device="cuda").bfloat16()
    b = torch.randn(n, device="cuda").bfloat16()
    for _ in range(2):                     # the second call finds the scratch as the first left it
        got = dot_sum(a, b)
    want = (a.double() * b.double()).sum()
    assert abs(float(got) - float(want)) <= 1e-3 * float((a.double() * b.double()).abs().sum().sqrt()) + 1e-3


@pytest.mark.parametrize("n,v,start", [(64, 1000, 0), (300, 25152, 25152), (7, 4099, 100)])
def test_cross_entropy_kernels_match_fp32(n, v, start):
    """One vocabulary shard alone (group of one): loss and gradient against torch's fp32 cross-entropy over the shard,
    with targets outside the shard and ignored rows."""
    from mesh_b200.parallel.vocab_ce import vocab_parallel_cross_entropy
    torch.manual_seed(0)
    logits = (torch.randn(n, v, device="cuda") * 3).bfloat16().requires_grad_(True)
    targets = torch.randint(start, start + v, (n,), device="cuda")
    targets[::5] = -100
    loss = vocab_parallel_cross_entropy(logits, targets, start, None, reduction="sum")
    loss.backward()
    ref = logits.detach().float().requires_grad_(True)
    local = torch.where(targets == -100, targets, targets - start)
    want = torch.nn.functional.cross_entropy(ref, local, ignore_index=-100, reduction="sum")
    want.backward()
    assert abs(float(loss) - float(want)) <= 2e-3 * abs(float(want)) + 1e-3
    assert float((logits.grad.float() - ref.grad).abs().max()) < 8e-3
