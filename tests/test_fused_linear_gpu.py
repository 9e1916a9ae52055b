"""Fused tensor-parallel linear layers (all-gather -> GEMM, GEMM -> reduce-scatter) against fp32 PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rank(rank, world, rdv):
    from mesh_b200.config import MeshConfig, set_config
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.parallel.fused_linear import FusedColumnLinear, FusedRowLinear, column_linear, row_linear
    from mesh_b200.utils.status import check_status
    torch.cuda.set_device(rank)
    set_config(MeshConfig.from_env(heap_bytes=1 << 30))
    ctx = MeshContext(rank, world, torch.device("cuda", rank), rdv, None)
    M, D, N = 256 * world, 512, 768                     # tokens, model width, projection width (all ranks together)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, D, generator=g).bfloat16()
    wc = (torch.randn(N, D, generator=g) * 0.05).bfloat16()      # column-parallel: rows cut
    wr = (torch.randn(D, N, generator=g) * 0.05).bfloat16()      # row-parallel: columns cut
    dy = torch.randn(M, D, generator=g).bfloat16()
    rows, Nl = M // world, N // world
    col = FusedColumnLinear(ctx.heap, M, D, Nl)
    row = FusedRowLinear(ctx.heap, M, Nl, D)
    for step in range(3):                                # several uses: the landing zones alternate
        xs = x[rank * rows:(rank + 1) * rows].cuda().requires_grad_(True)
        wcl = wc[rank * Nl:(rank + 1) * Nl].cuda().requires_grad_(True)
        wrl = wr[:, rank * Nl:(rank + 1) * Nl].contiguous().cuda().requires_grad_(True)
        h = column_linear(xs, wcl, col)                  # [M, Nl]
        y = row_linear(torch.tanh(h), wrl, row)          # [rows, D]
        y.backward(dy[rank * rows:(rank + 1) * rows].cuda())
        torch.cuda.synchronize()
        check_status()
        # reference on the whole problem in fp32
        xf, wcf, wrf = x.float().requires_grad_(True), wc.float().requires_grad_(True), wr.float().requires_grad_(True)
        hf = (xf @ wcf.T).to(torch.bfloat16).float()
        yf = torch.tanh(hf) @ wrf.T
        yf.backward(dy.float())

        def close(a, b, tol=3e-2):
            assert (a.float().cpu() - b).abs().max() <= tol * b.abs().max() + 1e-3, float((a.float().cpu() - b).abs().max() / b.abs().max())
        close(y, yf[rank * rows:(rank + 1) * rows].detach())
        close(xs.grad, xf.grad[rank * rows:(rank + 1) * rows])
        close(wcl.grad, wcf.grad[rank * Nl:(rank + 1) * Nl])
        close(wrl.grad, wrf.grad[:, rank * Nl:(rank + 1) * Nl])
    rdv.barrier("fused-linear-done")
    ctx.heap.close()


@pytest.mark.parametrize("world", [2, 4])
def test_fused_column_and_row_linear(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_rank, world, use_cuda=True, timeout=300.0)


def _rank_all_reduce(rank, world, rdv):
    from mesh_b200.config import MeshConfig, set_config
    from mesh_b200.distributed.comm import Communicator
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.parallel.fused_linear import FusedRowLinearAllReduce, row_linear_all_reduce
    from mesh_b200.utils.status import check_status
    torch.cuda.set_device(rank)
    set_config(MeshConfig.from_env(heap_bytes=1 << 30))
    ctx = MeshContext(rank, world, torch.device("cuda", rank), rdv, None)
    comm = Communicator(ctx.heap, staging_bytes=32 << 20, p2p_slot_bytes=8 << 20)
    M, D, N = 256 * world, 512, 768
    g = torch.Generator().manual_seed(4)
    h = torch.randn(M, N, generator=g).bfloat16()
    w = (torch.randn(D, N, generator=g) * 0.05).bfloat16()
    dy = torch.randn(M, D, generator=g).bfloat16()
    Nl = N // world
    op = FusedRowLinearAllReduce(ctx.heap, comm, M, Nl, D)
    for step in range(2):
        hl = h[:, rank * Nl:(rank + 1) * Nl].contiguous().cuda().requires_grad_(True)
        wl = w[:, rank * Nl:(rank + 1) * Nl].contiguous().cuda().requires_grad_(True)
        y = row_linear_all_reduce(hl, wl, op)                     # [M, D], whole on every rank
        y.backward(dy.cuda())
        torch.cuda.synchronize()
        check_status()
        hf, wf = h.float().requires_grad_(True), w.float().requires_grad_(True)
        yf = hf @ wf.T
        yf.backward(dy.float())

        def close(a, b, tol=3e-2):
            assert (a.float().cpu() - b).abs().max() <= tol * b.abs().max() + 1e-3
        close(y, yf.detach())
        close(hl.grad, hf.grad[:, rank * Nl:(rank + 1) * Nl])
        close(wl.grad, wf.grad[:, rank * Nl:(rank + 1) * Nl])
    rdv.barrier("fused-ar-done")
    ctx.heap.close()


def test_fused_row_linear_all_reduce():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_rank_all_reduce, 2, use_cuda=True, timeout=300.0)
