"""Error measures for kernels with bf16 outputs, against fp32 PyTorch statements of the same operation.

A bf16 value carries a relative rounding error of about 1.1e-3 RMS, so a correct kernel sits at a few 1e-3 of
RMS-relative error; a maximum-error bound relative to the largest reference value is far looser and lets a wrong
tile in a low-magnitude region pass.  ``assert_close_rms`` checks the whole matrix and every 128 x 256 tile of it."""
import torch


def rms_rel(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.float(), want.float()
    return float((got - want).square().mean().sqrt() / want.square().mean().sqrt().clamp_min(1e-20))


def assert_close_rms(got: torch.Tensor, want: torch.Tensor, tol: float = 4e-3, tile_tol: float | None = None,
                     tile=(128, 256), what: str = "") -> None:
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    got2 = got.float().reshape(-1, got.shape[-1])
    want2 = want.float().reshape(-1, want.shape[-1]).to(got2.device)
    assert torch.isfinite(got2).all(), f"{what}: non-finite values"
    e = rms_rel(got2, want2)
    assert e <= tol, f"{what}: RMS-relative error {e:.3e} > {tol:.1e}"
    tile_tol = 4 * tol if tile_tol is None else tile_tol
    scale = float(want2.square().mean().sqrt())
    tm, tn = tile
    M, N = got2.shape
    worst, where = 0.0, None
    for i in range(0, M, tm):
        d = (got2[i:i + tm] - want2[i:i + tm]).square()
        w = want2[i:i + tm].square()
        for j in range(0, N, tn):
            # a tile's error against the larger of its own and the matrix's magnitude: a tile of near-zero
            # reference values is not held to a relative bound it cannot meet
            ref = max(float(w[:, j:j + tn].mean().sqrt()), 0.05 * scale, 1e-20)
            t = float(d[:, j:j + tn].mean().sqrt()) / ref
            if t > worst:
                worst, where = t, (i, j)
    assert worst <= tile_tol, f"{what}: tile at {where} has RMS-relative error {worst:.3e} > {tile_tol:.1e}"
