"""Sharded checkpoint round trip with reshard on load, journal semantics, sharded AdamW vs torch.optim.AdamW."""
import json

import torch

from mesh_b200.ckpt import latest_step, load_sharded, save_sharded
from mesh_b200.compiler.placement import counts
from mesh_b200.parallel.optim import ShardedAdamW


def test_reshard_on_load(tmp_path):
    full = {"w": torch.arange(10 * 6, dtype=torch.float32).view(10, 6), "b": torch.arange(4.0)}
    lay4 = {"w": (0, counts(10, None, 4)), "b": (None, None)}
    for r in range(4):
        lo = sum(lay4["w"][1][:r])
        save_sharded(tmp_path, 3, {"w": full["w"][lo:lo + lay4["w"][1][r]], "b": full["b"]}, lay4, r, 4, extra={"lr": 0.1})
    assert latest_step(tmp_path) == 3
    for world in (1, 2, 3):
        got = [load_sharded(tmp_path, None, r, world)[0] for r in range(world)]
        assert torch.equal(torch.cat([g["w"] for g in got], 0), full["w"])
        assert all(torch.equal(g["b"], full["b"]) for g in got)
    unequal = {"w": (0, [7, 3])}
    a = load_sharded(tmp_path, 3, 0, 2, unequal)[0]["w"]
    assert a.shape[0] == 7 and torch.equal(a, full["w"][:7])
    # stored replicated, wanted cut: every rank gets its slice, not the whole tensor
    cut = {"b": (0, [1, 3])}
    assert torch.equal(load_sharded(tmp_path, 3, 0, 2, cut)[0]["b"], full["b"][:1])
    assert torch.equal(load_sharded(tmp_path, 3, 1, 2, cut)[0]["b"], full["b"][1:])
    # a step that began but never committed is ignored
    with open(tmp_path / "journal.jsonl", "a") as j:
        j.write(json.dumps({"event": "begin", "step": 9, "world": 4}) + "\n" + '{"event": "comm')
    assert latest_step(tmp_path) == 3


def test_sharded_adamw_matches_torch():
    torch.manual_seed(0)
    p_ref = torch.nn.Parameter(torch.randn(37, 5))
    p = torch.nn.Parameter(p_ref.detach().clone())
    ref = torch.optim.AdamW([p_ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt = ShardedAdamW([p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(5):
        g = torch.randn(37, 5)
        p_ref.grad = g.clone()
        ref.step()
        opt.step([g])
    assert torch.allclose(p, p_ref, atol=1e-6)
    sd = opt.state_dict()
    opt2 = ShardedAdamW([torch.nn.Parameter(p.detach().clone())], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    opt2.load_state_dict(sd)
    assert opt2.step_no == 5 and torch.equal(opt2.state[0]["m"], opt.state[0]["m"])


def test_reshard_round_trips_over_random_layouts(tmp_path):
    """Any old world and cut to any new world and cut (same dimension, another dimension, or replicated), with unequal
    shares and shards of size zero, gives back the same bytes and dtypes."""
    import random
    from mesh_b200.ckpt.sharded import load_sharded, save_sharded
    from mesh_b200.compiler.placement import counts
    random.seed(0)
    torch.manual_seed(0)
    for trial in range(25):
        shape = [random.randint(1, 7) for _ in range(random.randint(1, 3))]
        full = torch.randn(*shape).to(random.choice([torch.float32, torch.bfloat16]))
        ids = torch.arange(shape[0] * 2).reshape(shape[0], 2)
        ow, nw = random.randint(1, 5), random.randint(1, 5)
        dim = random.randrange(len(shape))
        oc = counts(shape[dim], random.choice([None, [random.randint(1, 4) for _ in range(ow)]]), ow)
        ic = counts(shape[0], None, ow)
        d = tmp_path / f"t{trial}"
        for r in range(ow):
            local = {"a": full.narrow(dim, sum(oc[:r]), oc[r]), "i": ids.narrow(0, sum(ic[:r]), ic[r]), "r": full.flatten()[:1]}
            save_sharded(d, 1, local, {"a": (dim, oc), "i": (0, ic), "r": (None, None)}, r, ow)
        ndim = random.choice([dim, dim, random.randrange(len(shape)), None])
        nc = counts(shape[ndim], random.choice([None, [random.randint(1, 4) for _ in range(nw)]]), nw) if ndim is not None else None
        parts = [load_sharded(d, None, r, nw, {"a": (ndim, nc)})[0] for r in range(nw)]
        got = torch.cat([p["a"] for p in parts], ndim) if ndim is not None else parts[-1]["a"]
        assert got.dtype == full.dtype and torch.equal(got, full), (shape, ow, nw, dim, ndim, oc, nc)
        assert torch.equal(torch.cat([p["i"] for p in parts], 0), ids) and parts[0]["i"].dtype == torch.int64
        assert all(torch.equal(p["r"], full.flatten()[:1]) for p in parts)
