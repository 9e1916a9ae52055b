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
