"""Expert-parallel MoE layer (fused dispatch / grouped tcgen05 GEMMs / combine) vs a dense fp32 PyTorch statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(got, want, tol):
    err = (got.float() - want.float()).abs().max().item()
    ref = want.float().abs().max().item() + 1e-6
    assert err / ref < tol, f"max err {err} vs {ref}"


def _run(rank, world, rdv, T, D, F, E, k, steps):
    from mesh_b200.config import MeshConfig, set_config
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.parallel.moe import EPMoE, moe_reference
    from mesh_b200.utils.status import check_status
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    set_config(MeshConfig.from_env(heap_bytes=512 << 20))
    ctx = MeshContext(rank, world, dev, rdv, None)
    g = torch.Generator(device="cpu").manual_seed(0)
    xs = [torch.randn(T, D, generator=g).bfloat16() for _ in range(world)]
    dys = [torch.randn(T, D, generator=g).bfloat16() for _ in range(world)]
    wr = (torch.randn(E, D, generator=g) * 0.1).bfloat16()
    w1 = (torch.randn(E, 2 * F, D, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(E, D, F, generator=g) * 0.05).bfloat16()
    bias = [torch.randn(E, generator=g) for _ in range(world)]          # per-rank bias: skewed, uneven loads
    El = E // world
    moe = EPMoE(ctx, T, D, F, E, k, capacity_factor=3.0)
    x, dy = xs[rank].to(dev), dys[rank].to(dev)
    w1l = w1[rank * El:(rank + 1) * El].reshape(El * 2 * F, D).contiguous().to(dev)
    w2l = w2[rank * El:(rank + 1) * El].reshape(El * D, F).contiguous().to(dev)
    wrd, bd = wr.to(dev), bias[rank].to(dev)
    for _ in range(steps):
        out = moe.forward(x, wrd, w1l, w2l, bd)
        dx, dwr, dw1, dw2 = moe.backward(dy)
    check_status()
    assert int(moe.layout[3 * El + 1]) == 0, "capacity overflow in the test configuration"
    # reference: all ranks' tokens through all experts, autograd for the gradients
    W1, W2, WR = w1.to(dev).float().requires_grad_(True), w2.to(dev).float().requires_grad_(True), wr.to(dev).float().requires_grad_(True)
    outs, xrs = [], []
    for r in range(world):
        xr = xs[r].to(dev).float().requires_grad_(True)
        outs.append(moe_reference(xr, WR, W1, W2, k, bias[r].to(dev)))
        xrs.append(xr)
    sum((o * dys[r].to(dev).float()).sum() for r, o in enumerate(outs)).backward()
    _close(out, outs[rank], 3e-2)
    _close(dx, xrs[rank].grad, 5e-2)
    _close(dw1.view(El, 2 * F, D), W1.grad[rank * El:(rank + 1) * El], 5e-2)
    _close(dw2.view(El, D, F), W2.grad[rank * El:(rank + 1) * El], 5e-2)
    rdv.barrier("moe-done")
    ctx.heap.close()


def test_moe_world1():
    import torch.distributed as dist
    from mesh_b200.runtime.rendezvous import Rendezvous
    _run(0, 1, Rendezvous(dist.HashStore(), 0, 1), 256, 256, 128, 8, 2, 2)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_moe_expert_parallel(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_run, world, 256, 256, 128, 8 * world // 2 if world > 2 else 8, 2, 2, use_cuda=True, timeout=300.0)
