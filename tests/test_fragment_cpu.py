"""``mesh::fragment``: the coded-tile dequantisation against its encoder, per-tile widths, export."""
import torch

from mesh_b200.ops.fragment import encode_fragment, fragment


def _decode_all(f, R, C, rows=None, cols=None):
    rows = torch.arange(R) if rows is None else rows
    cols = torch.arange(C) if cols is None else cols
    return fragment(f["codes"], f["tiles"], f["bands"], f["row_scale"], f["col_scale"], rows, cols, torch.float32)


def test_round_trip_within_half_a_level():
    torch.manual_seed(0)
    w = torch.randn(64, 96)
    for width in (3, 4, 7, 8, 11, 15):
        f = encode_fragment(w, width)
        got = _decode_all(f, 64, 96)
        # per tile: |error| <= half a quantisation step, plus the rounding of the tile scale to fp16 (2^-11 relative)
        amax = w.reshape(2, 32, 3, 32).abs().amax((1, 3))
        step = 2 * amax / (2 ** width - 1)
        err = (got - w).reshape(2, 32, 3, 32).abs().amax((1, 3))
        assert (err <= 0.5 * step * 1.01 + amax * 2 ** -10).all(), (width, err, step)


def test_levels_are_exact_and_zero_width_is_zero():
    # a matrix made of exact levels decodes bit for bit; width 0 tiles are zero; fields crossing 16 bits (width 5) work
    torch.manual_seed(1)
    widths = torch.tensor([[5, 0], [9, 4]])
    scale = 0.25
    w = torch.zeros(64, 64)
    for tr in range(2):
        for tc in range(2):
            wd = int(widths[tr, tc])
            if wd:
                sym = torch.randint(0, 2 ** wd, (32, 32))
                sym[0, 0], sym[0, 1] = 2 ** wd - 1, 0            # make the extreme levels appear: fixes the scale
                w[tr * 32:(tr + 1) * 32, tc * 32:(tc + 1) * 32] = (2 * sym + 1 - 2 ** wd) * 0.5 * scale
    f = encode_fragment(w, widths)
    got = _decode_all(f, 64, 64)
    assert torch.equal(got[:32, 32:], torch.zeros(32, 32))
    assert torch.allclose(got, w, rtol=2e-3, atol=0)             # tile scale is stored as fp16
    # row / column selections and scales
    f["row_scale"] = torch.linspace(0.5, 2, 64)
    f["col_scale"] = torch.linspace(1, 3, 64)
    rows, cols = torch.tensor([63, 0, 17]), torch.tensor([5, 40, 41, 2])
    sub = _decode_all(f, 64, 64, rows, cols)
    want = (got * f["row_scale"][:, None] * f["col_scale"][None, :])[rows][:, cols]
    assert torch.allclose(sub, want, rtol=1e-6)


def test_fragment_exports():
    w = torch.randn(32, 32)
    f = encode_fragment(w, 4)

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            for k, v in f.items():
                self.register_buffer(k, v)

        def forward(self, x):
            wt = torch.ops.mesh.fragment(self.codes, self.tiles, self.bands, self.row_scale, self.col_scale,
                                         torch.arange(32), torch.arange(32), torch.float32)
            return x @ wt.T

    ep = torch.export.export(M(), (torch.randn(3, 32),))
    assert any("fragment" in str(n.target) for n in ep.graph.nodes)
    x = torch.randn(3, 32)
    assert torch.allclose(ep.module()(x), M()(x))


def test_coded_matrix_transforms_selection_and_file_round_trip(tmp_path):
    from mesh_b200.ops.fragment import CodedFFN, CodedMatrix, hadamard_transform, load_matrices, save_matrices
    torch.manual_seed(3)
    R, C = 64, 64
    w = torch.randn(R, C) / 8
    x = torch.randn(5, C)
    # plain
    plain = CodedMatrix(encode_fragment(w, 8))
    assert (plain(x) - x @ w.T).abs().max() < 0.05
    # sign flip + Hadamard: code W H^-1 so that (H s x) W'^T = x W^T
    signs = torch.where(torch.rand(C) < 0.5, -1.0, 1.0)
    Hm = hadamard_transform(torch.eye(C)) / C ** 0.5                 # orthonormal, symmetric
    w_rot = (w * signs[None, :]) @ Hm.T                              # W diag(s) H^T
    f = encode_fragment(w_rot, 8)
    f["signs"] = signs
    mixed = CodedMatrix(f)
    assert (mixed(x) - x @ w.T).abs().max() < 0.05
    # a dense rotation
    q, _ = torch.linalg.qr(torch.randn(C, C))
    f = encode_fragment(w @ q.T, 8)
    f["rotation"], f["rotation_scale"] = q, torch.ones(C)
    rot = CodedMatrix(f)
    assert (rot(x) - x @ w.T).abs().max() < 0.05
    # row / column selection = the same slice of the dense product
    sub = plain.select(rows=torch.arange(32, 64), columns=torch.arange(0, 32))
    assert (sub(x[:, :32]) - x[:, :32] @ w[32:, :32].T).abs().max() < 0.05
    # FFN share and file round trip
    wg, wu, wd = torch.randn(64, 64) / 8, torch.randn(64, 64) / 8, torch.randn(64, 64) / 8
    mats = {"gate": encode_fragment(wg, 8), "up": encode_fragment(wu, 8), "down": encode_fragment(wd, 8)}
    save_matrices(tmp_path / "ffn.safetensors", mats)
    loaded = load_matrices(tmp_path / "ffn.safetensors")
    ffn = CodedFFN(loaded["gate"], loaded["up"], loaded["down"], first=32, count=32)
    ref = (torch.nn.functional.gelu(x @ wg[32:].T, approximate="tanh") * (x @ wu[32:].T)) @ wd[:, 32:].T
    assert ffn.shared and (ffn(x) - ref).abs().max() < 0.1
