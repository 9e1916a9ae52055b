"""The stock arm of the hybrid benchmark: every grid gives the loss and the update of its own single-process run."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _cfg():
    from baseline.hybrid_stock import StockConfig
    return StockConfig(vocab=64, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64, seq_len=16)


def _data(dp_rank, M=2):
    g = torch.Generator().manual_seed(5 + dp_rank)
    return torch.randint(0, 64, (M, 16), generator=g), torch.randint(0, 64, (M, 16), generator=g)


def _solo():
    from baseline.hybrid_stock import Grid, StockTrainer
    tr = StockTrainer(_cfg(), Grid("", 0, 1), torch.device("cpu"), torch.float32, micro_batch=1, n_micro=2, lr=1e-2)
    losses = [float(tr.step(*_data(0))) for _ in range(2)]
    return losses, tr.stage.blocks[0].w_2.detach().clone(), tr.stage.embed.detach().clone()


def _rank(rank, world, rdv, grid_text):
    from baseline.hybrid_stock import Grid, StockTrainer
    torch.manual_seed(0)
    grid = Grid(grid_text, rank, world)
    tr = StockTrainer(_cfg(), grid, torch.device("cpu"), torch.float32, micro_batch=1, n_micro=2, lr=1e-2)
    losses = [float(tr.step(*_data(grid.coord["dp"]))) for _ in range(2)]
    ref_losses, ref_w2, ref_embed = _solo()
    if grid.size["dp"] == 1:
        assert max(abs(a - b) for a, b in zip(losses, ref_losses)) < 1e-4, (losses, ref_losses)
        if tr.stage.first:
            assert torch.allclose(tr.stage.embed, ref_embed, atol=1e-4)
        if grid.coord["pp"] == 0:
            cols = ref_w2.shape[1] // grid.size["tp"]
            mine = ref_w2[:, grid.coord["tp"] * cols:(grid.coord["tp"] + 1) * cols]
            assert torch.allclose(tr.stage.blocks[0].w_2, mine, atol=1e-4)
    else:
        assert all(l == l and l > 0 for l in losses)


@pytest.mark.parametrize("grid", ["tp2", "cp2", "pp2", "dp2"])
def test_stock_arm_matches_its_single_process_run(grid):
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_rank, 2, grid, init_pg="gloo")
