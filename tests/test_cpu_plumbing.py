"""CPU/gloo fake cluster: the ``mesh`` backend's CPU half and the TP2 SwiGLU FFN plumbing check
(fp32 x[128,1024], 1024->4096->1024, one all-reduce on the output, must match the single-device FFN
to 1e-5 relative)."""
import torch
import torch.distributed as dist

from mesh_b200.utils.launch import spawn_ranks


def _pg_rank(rank, world, rdv):
    import mesh_b200.distributed.process_group  # noqa: F401  (registers "mesh")
    import os
    dist.init_process_group("mesh", rank=rank, world_size=world,
                            init_method=f"tcp://127.0.0.1:{os.environ['MESH_AUX_PORT']}")
    try:
        t = torch.full((5,), float(rank + 1))
        dist.all_reduce(t)
        assert torch.allclose(t, torch.full((5,), float(sum(range(1, world + 1)))))
        out = torch.empty(world * 3)
        dist.all_gather_into_tensor(out, torch.full((3,), float(rank)))
        assert out.tolist() == [float(r) for r in range(world) for _ in range(3)]
        rs = torch.empty(2)
        dist.reduce_scatter_tensor(rs, torch.arange(world * 2, dtype=torch.float32))
        assert torch.allclose(rs, torch.arange(world * 2, dtype=torch.float32)[rank * 2:rank * 2 + 2] * world)
        b = torch.tensor([float(rank)])
        dist.broadcast(b, src=1)
        assert b.item() == 1.0
        a2a = torch.empty(world)
        dist.all_to_all_single(a2a, torch.arange(world, dtype=torch.float32) + 10 * rank)
        assert a2a.tolist() == [float(rank + 10 * r) for r in range(world)]
        if rank == 0:
            dist.send(torch.tensor([42.0]), dst=1)
        elif rank == 1:
            r = torch.zeros(1)
            dist.recv(r, src=0)
            assert r.item() == 42.0
        dist.barrier()
        assert dist.get_backend() == "mesh"
    finally:
        dist.destroy_process_group()


def test_mesh_backend_cpu_delegate():
    spawn_ranks(_pg_rank, 3)


def _ffn_rank(rank, world, rdv):
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.parallel.layers import TPGatedFFN
    ctx = MeshContext(rank, world, torch.device("cpu"), rdv, dist.group.WORLD)
    torch.manual_seed(0)
    x = torch.randn(128, 1024)
    dy = torch.randn(128, 1024)
    # unsharded reference: the same module as a world of one
    solo = TPGatedFFN(1024, 4096, MeshContext(0, 1, torch.device("cpu"), rdv, None), dtype=torch.float32, seed=3,
                      sequence_parallel=False)
    xs = x.clone().requires_grad_(True)
    ys = solo(xs)
    ys.backward(dy)
    # TP2, replicated activations, ONE all-reduce on the output
    tp = TPGatedFFN(1024, 4096, ctx, dtype=torch.float32, seed=3, sequence_parallel=False)
    xt = x.clone().requires_grad_(True)
    yt = tp(xt)
    yt.backward(dy)
    rel = (yt - ys).abs().max() / ys.abs().max()
    assert rel < 1e-5, rel
    assert (xt.grad - xs.grad).abs().max() / xs.grad.abs().max() < 1e-5
    Fl = 4096 // world
    assert torch.allclose(tp.w_down.grad, solo.w_down.grad[:, rank * Fl:(rank + 1) * Fl], rtol=1e-4, atol=1e-5)
    # sequence-parallel form: all-gather in, reduce-scatter out
    sp = TPGatedFFN(1024, 4096, ctx, dtype=torch.float32, seed=3, sequence_parallel=True)
    rows = 128 // world
    ysp = sp(x[rank * rows:(rank + 1) * rows])
    assert (ysp - ys[rank * rows:(rank + 1) * rows]).abs().max() / ys.abs().max() < 1e-5


    # unequal shares of the hidden units (a rank three times the other): the same layer
    shares = [3072, 1024]
    un = TPGatedFFN(1024, 4096, ctx, dtype=torch.float32, seed=3, sequence_parallel=True, ff_shares=shares)
    assert un.w_down.shape == (1024, shares[rank])
    yun = un(x[rank * rows:(rank + 1) * rows])
    assert (yun - ys[rank * rows:(rank + 1) * rows]).abs().max() / ys.abs().max() < 1e-5


def test_tp2_swiglu_ffn_matches_single_device():
    spawn_ranks(_ffn_rank, 2, init_pg="gloo")


def _dp_rank(rank, world, rdv):
    from mesh_b200.parallel.dp import DataParallel
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
    ref = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
    ref.load_state_dict(m.state_dict())
    g = torch.Generator().manual_seed(1)
    x = torch.randn(8 * world, 16, generator=g)
    dp = DataParallel(m, world, rank, bucket_bytes=1024)
    m(x[rank * 8:(rank + 1) * 8]).pow(2).mean().backward()
    dp.finish()
    ref(x).pow(2).mean().backward()                       # the full batch on one device
    for a, b in zip(m.parameters(), ref.parameters()):
        assert torch.allclose(a.grad, b.grad, atol=1e-6)


def test_data_parallel_overlapped_reduce_scatter_matches_full_batch():
    spawn_ranks(_dp_rank, 2, init_pg="gloo")


def _zero1_rank(rank, world, rdv):
    """Bucketed ZeRO-1: DataParallel's per-bucket reduce-scatter + BucketedAdamW against torch.optim.AdamW on the
    full batch, several steps."""
    from mesh_b200.parallel.dp import DataParallel
    from mesh_b200.parallel.optim import BucketedAdamW
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(16, 33), torch.nn.Tanh(), torch.nn.Linear(33, 5))
    ref = torch.nn.Sequential(torch.nn.Linear(16, 33), torch.nn.Tanh(), torch.nn.Linear(33, 5))
    ref.load_state_dict(m.state_dict())
    dp = DataParallel(m, world, rank, bucket_bytes=512, all_reduce=False)
    assert len(dp.buckets) >= 2
    opt = BucketedAdamW(dp, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    g = torch.Generator().manual_seed(1)
    for step in range(4):
        x = torch.randn(8 * world, 16, generator=g)
        for p in m.parameters():
            p.grad = None
        m(x[rank * 8:(rank + 1) * 8]).pow(2).mean().backward()
        opt.step()
        ropt.zero_grad()
        ref(x).pow(2).mean().backward()
        ropt.step()
    for a, b in zip(m.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=2e-5), float((a - b).abs().max())


def test_bucketed_zero1_optimizer_matches_adamw_on_the_full_batch():
    spawn_ranks(_zero1_rank, 2, init_pg="gloo")
