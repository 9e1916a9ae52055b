"""Vocabulary-parallel cross-entropy against ``F.cross_entropy`` on the gathered logits (gloo ranks)."""
import torch
import torch.nn.functional as F


def _rank(rank, world, rdv):
    import torch.distributed as dist
    from mesh_b200.parallel.vocab_ce import VocabParallelHead, vocab_parallel_cross_entropy
    g = torch.Generator().manual_seed(0)
    n, v = 12, 32
    logits = torch.randn(n, v, generator=g) * 3
    targets = torch.randint(0, v, (n,), generator=g)
    targets[3] = -100
    ref_in = logits.clone().requires_grad_(True)
    ref = F.cross_entropy(ref_in, targets, ignore_index=-100)
    ref.backward()
    cols = v // world
    mine = logits[:, rank * cols:(rank + 1) * cols].clone().requires_grad_(True)
    loss = vocab_parallel_cross_entropy(mine, targets, rank * cols, dist.group.WORLD)
    loss.backward()
    assert abs(float(loss) - float(ref)) < 1e-5
    assert torch.allclose(mine.grad, ref_in.grad[:, rank * cols:(rank + 1) * cols], atol=1e-6)
    per_token = vocab_parallel_cross_entropy(mine.detach(), targets, rank * cols, dist.group.WORLD, reduction="none")
    assert torch.allclose(per_token, F.cross_entropy(logits, targets, ignore_index=-100, reduction="none"), atol=1e-5)
    # the head: hidden states replicated, weight rows cut; gradients of h are summed over the axis
    h = torch.randn(n, 16, generator=g)
    head = VocabParallelHead(16, v, rank, world, dist.group.WORLD)
    full_w = torch.empty(v, 16).normal_(0, 0.02, generator=torch.Generator().manual_seed(7)).requires_grad_(True)
    hp, hf = h.clone().requires_grad_(True), h.clone().requires_grad_(True)
    lp, lf = head(hp, targets), F.cross_entropy(F.linear(hf, full_w), targets, ignore_index=-100)
    lp.backward()
    lf.backward()
    assert abs(float(lp) - float(lf)) < 1e-5 and torch.allclose(hp.grad, hf.grad, atol=1e-6)
    assert torch.allclose(head.weight.grad, full_w.grad[rank * cols:(rank + 1) * cols], atol=1e-6)


def test_vocab_parallel_cross_entropy_two_and_four_ranks():
    from mesh_b200.utils.launch import spawn_ranks
    for world in (2, 4):
        spawn_ranks(_rank, world, init_pg="gloo")
