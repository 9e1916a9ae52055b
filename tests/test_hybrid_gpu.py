"""Hybrid parallel training step on GPUs (bf16, this package's kernels) against the fp32 single-process model."""
import pytest
import torch
import torch.distributed as dist

from mesh_b200.parallel.topology import ParallelDims

pytestmark = pytest.mark.gpu


def _rank(rank, world, rdv, dims_text):
    from mesh_b200.config import MeshConfig, set_config
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.models.hybrid import HybridConfig, HybridTrainer, reference_loss_and_grads
    from mesh_b200.parallel.topology import ParallelContext
    from mesh_b200.utils.status import check_status
    torch.cuda.set_device(rank)
    set_config(MeshConfig.from_env(heap_bytes=2 << 30))
    dims = ParallelDims.parse(dims_text)
    ctx = MeshContext(rank, world, torch.device("cuda", rank), rdv, dist.group.WORLD if world > 1 else None)
    par = ParallelContext(ctx, dims)
    cfg = HybridConfig(vocab=512, d_model=512, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=128, d_ff=1024, seq_len=512,
                       init_std=0.05)
    mb, M = 1, 2
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, cfg.vocab, (dims.dp * mb * M, cfg.seq_len), generator=g)
    targets = torch.randint(0, cfg.vocab, (dims.dp * mb * M, cfg.seq_len), generator=g)
    tr = HybridTrainer(cfg, par, micro_batch=mb, n_micro=M, lr=2e-3)
    d = par.dp.rank
    tok, tgt = tokens[d * mb * M:(d + 1) * mb * M].cuda(), targets[d * mb * M:(d + 1) * mb * M].cuda()
    losses = [float(tr.step(tok, tgt)) for _ in range(3)]
    torch.cuda.synchronize()
    check_status()
    ref_loss, _, _ = reference_loss_and_grads(cfg, tokens, targets)
    assert abs(losses[0] - ref_loss) < 3e-2 * ref_loss, (losses, ref_loss)
    assert losses[2] < losses[0], losses
    rdv.barrier("hybrid-done")
    if world > 1:
        ctx.heap.close()


@pytest.mark.parametrize("dims", ["solo", "tp2", "cp2", "pp2", "dp2", "tp2cp2", "tp2cp2pp2"])
def test_hybrid_training_step(dims):
    world = ParallelDims.parse(dims).world
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_rank, world, dims, use_cuda=True, timeout=300.0, init_pg="nccl" if world > 1 else None)
