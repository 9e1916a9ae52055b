"""Hybrid tensor x context x pipeline x data parallel training step on gloo ranks against the single-process model."""
import pytest
import torch
import torch.distributed as dist

from mesh_b200.parallel.topology import ParallelDims
from mesh_b200.utils.launch import spawn_ranks


def test_parallel_dims_grid():
    d = ParallelDims(dp=2, pp=2, cp=2, tp=2)
    assert d.world == 16
    assert d.coords(0) == {"tp": 0, "cp": 0, "pp": 0, "dp": 0}
    assert d.coords(13) == {"tp": 1, "cp": 0, "pp": 1, "dp": 1}
    assert d.rank_of(tp=1, cp=0, pp=1, dp=1) == 13
    assert d.axis_ranks(13, "tp") == [12, 13]
    assert d.axis_ranks(13, "cp") == [13, 15]
    assert d.axis_ranks(13, "pp") == [9, 13]
    assert d.axis_ranks(13, "dp") == [5, 13]
    groups = d.groups("cp")
    assert len(groups) == 8 and sorted(sum(groups, [])) == list(range(16))
    assert str(ParallelDims.parse("tp2 cp2 pp2")) == "tp2xcp2xpp2"
    assert ParallelDims.parse("dp8") == ParallelDims(dp=8)


def _pp_rank(rank, world, rdv, n_micro):
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.parallel.pp import run_1f1b
    from mesh_b200.parallel.topology import ParallelContext
    par = ParallelContext(MeshContext(rank, world, torch.device("cpu"), rdv, dist.group.WORLD), ParallelDims(pp=world))
    torch.manual_seed(0)
    layers = [torch.nn.Linear(16, 16) for _ in range(world)]
    xs = [torch.randn(4, 16) for _ in range(n_micro)]
    ts = [torch.randn(4, 16) for _ in range(n_micro)]
    mine = layers[rank]
    losses, stats = run_1f1b(lambda x: torch.tanh(mine(x)), par.pp, xs, act_shape=(4, 16), act_dtype=torch.float32,
                             loss_fn=lambda y, t: (y - t).pow(2).mean(), targets=ts)
    assert stats["peak_alive"] <= min(world - rank, n_micro)
    # the whole chain on one process
    ref = [torch.nn.Linear(16, 16) for _ in range(world)]
    for a, b in zip(ref, layers):
        a.load_state_dict(b.state_dict())
    tot = 0
    for x, t in zip(xs, ts):
        h = x
        for l in ref:
            h = torch.tanh(l(h))
        tot = tot + (h - t).pow(2).mean() / n_micro
    tot.backward()
    assert torch.allclose(mine.weight.grad, ref[rank].weight.grad, atol=1e-6)
    if rank == world - 1:
        assert abs(float(torch.stack(losses).mean()) - float(tot)) < 1e-6


@pytest.mark.parametrize("world,n_micro", [(2, 4), (4, 6), (3, 2)])
def test_1f1b_matches_single_process(world, n_micro):
    spawn_ranks(_pp_rank, world, n_micro, init_pg="gloo")


def _hybrid_rank(rank, world, rdv, dims_text, striped):
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.models.hybrid import HybridConfig, HybridTrainer, reference_loss_and_grads
    from mesh_b200.parallel.topology import ParallelContext
    dims = ParallelDims.parse(dims_text)
    par = ParallelContext(MeshContext(rank, world, torch.device("cpu"), rdv, dist.group.WORLD), dims)
    cfg = HybridConfig(vocab=64, d_model=32, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64, seq_len=16,
                       striped=striped, init_std=0.2)
    mb, M = 1, 2
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, cfg.vocab, (dims.dp * mb * M, cfg.seq_len), generator=g)
    targets = torch.randint(0, cfg.vocab, (dims.dp * mb * M, cfg.seq_len), generator=g)
    tr = HybridTrainer(cfg, par, micro_batch=mb, n_micro=M, dtype=torch.float32)
    d = par.dp.rank
    loss = tr.forward_backward(tokens[d * mb * M:(d + 1) * mb * M], targets[d * mb * M:(d + 1) * mb * M])
    ref_loss, ref_grads, ref = reference_loss_and_grads(cfg, tokens, targets)
    assert abs(float(loss) - ref_loss) < 1e-4 * max(1.0, abs(ref_loss)), (float(loss), ref_loss)
    # gradients: sum over dp of this rank's shard equals the reference's shard
    names = dict(tr.stage.named_parameters())
    lo = tr.stage.layers_range.start
    t, T = par.tp.rank, par.tp.world
    for name, p in names.items():
        gsum = p.grad.clone()
        if par.dp.world > 1:
            dist.all_reduce(gsum, group=par.dp.group)
        rname = name
        if name.startswith("blocks."):
            i = int(name.split(".")[1])
            rname = f"blocks.{lo + i}." + name.split(".", 2)[2]
        full = ref_grads[rname]
        if name.endswith("w_qkv"):
            hq, hk, hd = cfg.n_heads // T, cfg.n_kv_heads // T, cfg.head_dim
            q, k, v = full.split([cfg.n_heads * hd, cfg.n_kv_heads * hd, cfg.n_kv_heads * hd])
            want = torch.cat([q[t * hq * hd:(t + 1) * hq * hd], k[t * hk * hd:(t + 1) * hk * hd], v[t * hk * hd:(t + 1) * hk * hd]])
        elif name.endswith("w_o"):
            n = full.shape[1] // T
            want = full[:, t * n:(t + 1) * n]
        elif name.endswith("w_gate_up"):
            Fl = cfg.d_ff // T
            gate, up = full[: cfg.d_ff], full[cfg.d_ff:]
            want = torch.cat([gate[t * Fl:(t + 1) * Fl], up[t * Fl:(t + 1) * Fl]])
        elif name.endswith("w_down"):
            n = full.shape[1] // T
            want = full[:, t * n:(t + 1) * n]
        else:
            want = full
        err = (gsum - want).abs().max() / (want.abs().max() + 1e-12)
        assert err < 2e-4, (name, float(err))
    # and the optimiser step runs
    tr.opt.step()


@pytest.mark.parametrize("dims,striped", [("tp2", True), ("cp2", True), ("cp2", False), ("pp2", True), ("dp2", True),
                                          ("tp2cp2pp2", True)])
def test_hybrid_step_matches_single_process(dims, striped):
    spawn_ranks(_hybrid_rank, ParallelDims.parse(dims).world, dims, striped, init_pg="gloo")


def _ulysses_rank(rank, world, rdv):
    from mesh_b200.ops.attention import attention_ref, ulysses_attention
    from mesh_b200.parallel.topology import AxisContext
    axis = AxisContext("cp", rank, list(range(world)), torch.device("cpu"), dist.group.WORLD)
    g = torch.Generator().manual_seed(4)
    B, T, H, Hkv, hd = 2, 8 * world, 2 * world, world, 8
    q = torch.randn(B, T, H, hd, generator=g)
    k, v = torch.randn(B, T, Hkv, hd, generator=g), torch.randn(B, T, Hkv, hd, generator=g)
    dout = torch.randn(B, T, H, hd, generator=g)
    sl = slice(rank * (T // world), (rank + 1) * (T // world))
    ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
    o = ulysses_attention(ql, kl, vl, axis, causal=True)
    o.backward(dout[:, sl])
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref, _ = attention_ref(qf, kf, vf, True)
    ref.backward(dout)
    assert torch.allclose(o, ref[:, sl], atol=1e-5)
    for got, want in ((ql.grad, qf.grad), (kl.grad, kf.grad), (vl.grad, vf.grad)):
        assert torch.allclose(got, want[:, sl], atol=1e-5)


@pytest.mark.parametrize("world", [2, 4])
def test_head_exchange_attention_matches_full_attention(world):
    spawn_ranks(_ulysses_rank, world, init_pg="gloo")
