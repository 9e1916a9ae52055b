"""Fused all-gather->GEMM and GEMM->reduce-scatter FFN against the unsharded fp32 FFN."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _full_problem(M, D, F, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(M, D, generator=g)
    wg = torch.randn(F, D, generator=g) * 0.05
    wu = torch.randn(F, D, generator=g) * 0.05
    wd = torch.randn(D, F, generator=g) * 0.05
    dy = torch.randn(M, D, generator=g)
    return [t.bfloat16() for t in (x, wg, wu, wd, dy)]


def _reference(x, wg, wu, wd, dy):
    xr, wgr, wur, wdr = (t.float().cuda().requires_grad_(True) for t in (x, wg, wu, wd))
    y = (torch.nn.functional.silu(xr @ wgr.T) * (xr @ wur.T)) @ wdr.T
    y.backward(dy.float().cuda())
    return y.detach(), xr.grad, wgr.grad, wur.grad, wdr.grad


def _close(got, want, tol=8e-3):
    # intermediates (h, [g|u], [dg|du]) are rounded to bf16 on the way, the reference keeps fp32 throughout
    from _oracle import assert_close_rms
    assert_close_rms(got, want, tol=tol)


def _run_rank(rank, world, rdv, M, D, F, steps, shares=None):
    from mesh_b200.parallel.tp_ffn import FusedTPFFN
    from mesh_b200.runtime.heap import SymmetricHeap
    from mesh_b200.utils.status import check_status
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    heap = SymmetricHeap(rdv, 256 << 20, rank)
    x, wg, wu, wd, dy = _full_problem(M, D, F)
    y_ref, dx_ref, dwg_ref, dwu_ref, dwd_ref = _reference(x, wg, wu, wd, dy)
    rows = M // world
    shares = list(shares) if shares else [F // world] * world          # hidden units per rank
    Fl = shares[rank]
    sl = slice(rank * rows, (rank + 1) * rows)
    fs = slice(sum(shares[:rank]), sum(shares[:rank + 1]))
    wgu_l = torch.cat([wg[fs], wu[fs]], 0).to(dev)
    wd_l = wd[:, fs].contiguous().to(dev)
    x_l, dy_l = x[sl].to(dev), dy[sl].to(dev)
    op = FusedTPFFN(heap, M, D, F, ff_local=Fl)
    for _ in range(steps):   # repeated steps exercise the parity buffers and monotonic counters
        y = op.forward(x_l, wgu_l, wd_l)
        dx, dwgu, dwd = op.backward(dy_l)
    check_status()
    _close(y, y_ref[sl])
    _close(dx, dx_ref[sl])
    _close(dwgu[:Fl], dwg_ref[fs])
    _close(dwgu[Fl:], dwu_ref[fs])
    _close(dwd, dwd_ref[:, fs])
    rdv.barrier("done")
    heap.close()


def test_fused_tp_ffn_world1():
    import torch.distributed as dist
    from mesh_b200.runtime.rendezvous import Rendezvous
    rdv = Rendezvous(dist.HashStore(), 0, 1)
    _run_rank(0, 1, rdv, 512, 256, 512, 3)


def test_fused_tp_ffn_world1_many_waves():
    """Enough tiles for several waves per launch, so that the chained launches of a pass really overlap."""
    import torch.distributed as dist
    from mesh_b200.runtime.rendezvous import Rendezvous
    rdv = Rendezvous(dist.HashStore(), 0, 1)
    _run_rank(0, 1, rdv, 2048, 1024, 4096, 2)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_tp_ffn_multi(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_run_rank, world, 128 * world * 2, 256, 64 * world * 2, 3, use_cuda=True, timeout=300.0)
    spawn_ranks(_run_rank, world, 4096, 1024, 1792 * world, 2, use_cuda=True, timeout=300.0)


def test_fused_tp_ffn_unequal_hidden_shares():
    """Two ranks with different shares of the hidden units (1024 and 512 of 1536): the same kernels, the same numbers."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_run_rank, 2, 1024, 512, 1536, 2, (1024, 512), use_cuda=True, timeout=300.0)
