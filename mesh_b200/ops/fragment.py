"""Coded (quantised) weight matrices: the ``mesh::fragment`` operator and layers on top of it.

The operator keeps the name and signature of the reference's custom op
(``mesh::fragment(codes, tiles, bands, row_scale, col_scale, rows, columns, dtype) -> Tensor``, rdma/mesh_code.py:9-16;
dequantisation rule compiler/mesh_compiler/operations.py:6996-7040): a weight matrix is cut into 32x32 tiles, each with
its own bit width (0..15), a 12-bit offset into its band of packed 32-bit words and an fp16 scale; values are odd-integer
levels ``(2*symbol + 1 - 2^width) / 2`` times tile, row and column scales.  Here it is stated with tensor arithmetic
(it runs on CPU and CUDA tensors and under ``torch.export``), together with an encoder for round trips.

The production decode path of this package does not use that format: its kernels read 4-bit codes with one fp16 scale
per group of 64 inputs (``mesh_b200/csrc/ops/decode_linear.cu``), which is what :class:`CodedLinear` stores.  A
``fragment``-coded matrix can be converted once with :func:`to_group64`.
"""
from __future__ import annotations

import torch

_LIB = torch.library.Library("mesh", "FRAGMENT")
_LIB.define("fragment(Tensor codes, Tensor tiles, Tensor bands, Tensor row_scale, Tensor col_scale, "
            "Tensor rows, Tensor columns, ScalarType dtype) -> Tensor")
fragment = torch.ops.mesh.fragment.default


def _positions(device):
    """Per position (rr, cc) of a 32x32 tile: lane, bit-field index ``pair`` and which 16-bit half of the word."""
    rr = torch.arange(32, device=device)[:, None].expand(32, 32)
    cc = torch.arange(32, device=device)[None, :].expand(32, 32)
    lane = ((rr // 8) & 1) | ((cc & 3) << 1) | (((rr // 8) & 2) << 2) | ((cc & 4) << 2)
    pair = (rr & 6) * 2 + cc // 8
    half = (rr & 1) * 16
    return lane, pair, half


def _decode(codes, tiles, bands, row_scale, col_scale, rows, columns, dtype):
    dev = codes.device
    rows, columns = rows.to(dev, torch.int64), columns.to(dev, torch.int64)
    if codes.numel() == 0:
        return torch.zeros((rows.numel(), columns.numel()), dtype=dtype, device=dev)
    words = tiles.to(torch.int64) & 0xFFFFFFFF                               # [tile rows, tile cols]
    tile_scale = tiles.view(torch.float16)[..., 1::2].float()                 # the word's high half, as fp16
    r, c = rows[:, None], columns[None, :]
    rr, cc, tr, tc = r % 32, c % 32, r // 32, c // 32
    word = words[tr, tc]
    width = (word >> 12) & 15
    lane = ((rr // 8) & 1) | ((cc & 3) << 1) | (((rr // 8) & 2) << 2) | ((cc & 4) << 2)
    pair = (rr & 6) * 2 + cc // 8
    bit = pair * width
    shift, half = bit % 16, (rr & 1) * 16
    base = (bands.to(torch.int64)[tr] & 0x0FFFFFFF) + (word & 0xFFF)
    at = (base + bit // 16) * 32 + lane
    live = width != 0
    flat = codes.reshape(-1).to(torch.int64) & 0xFFFFFFFF
    n = flat.numel()
    low = torch.where(live, flat[at.clamp(0, n - 1)], torch.zeros_like(at))
    crossing = live & (shift + width > 16)
    high = torch.where(crossing, flat[(at + 32).clamp(0, n - 1)], torch.zeros_like(at))
    low, high = (low >> half) & 0xFFFF, (high >> half) & 0xFFFF
    joined = low | (high << 16)
    power = torch.ones_like(width) << width
    symbol = (joined >> shift) & (power - 1)
    odd = (2 * symbol + 1 - power).float()
    value = torch.where(live, odd * 0.5 * tile_scale[tr, tc], torch.zeros((), device=dev))
    value = value * row_scale.float()[rows][:, None] * col_scale.float()[columns][None, :]
    return value.to(dtype)


torch.library.impl(_LIB, "fragment", "CompositeExplicitAutograd")(_decode)


@torch.library.register_fake("mesh::fragment")
def _fragment_fake(codes, tiles, bands, row_scale, col_scale, rows, columns, dtype):
    return torch.empty((rows.numel(), columns.numel()), device=codes.device, dtype=dtype)


def encode_fragment(weight: torch.Tensor, width: int | torch.Tensor = 4):
    """Quantise ``weight [R, C]`` (R, C multiples of 32) into the fields of :func:`fragment`.

    ``width``: bits per value, one number or a ``[R/32, C/32]`` tensor of per-tile widths (0 = the tile is all zero).
    Row and column scales are 1; the tile scale is chosen so that the largest level covers the tile's largest value.
    Returns ``dict(codes, tiles, bands, row_scale, col_scale)``."""
    R, C = weight.shape
    assert R % 32 == 0 and C % 32 == 0
    TR, TC = R // 32, C // 32
    w = weight.detach().float().cpu()
    widths = torch.full((TR, TC), int(width), dtype=torch.int64) if not torch.is_tensor(width) else width.to(torch.int64).cpu()
    assert int(widths.max()) <= 15 and int(widths.min()) >= 0
    t = w.reshape(TR, 32, TC, 32).permute(0, 2, 1, 3)                        # [TR, TC, 32, 32]
    amax = t.abs().amax((-1, -2))
    levels = (torch.ones_like(widths) << widths) - 1                          # the largest odd level, 2^w - 1
    scale = torch.where((widths > 0) & (amax > 0), 2 * amax / levels.clamp(min=1).float(), torch.ones_like(amax))
    scale = scale.to(torch.float16)
    scale = torch.where(scale.float() > 0, scale, torch.ones_like(scale))
    power = torch.ones_like(widths) << widths
    sym = torch.round((t / (0.5 * scale.float())[..., None, None] + power[..., None, None].float() - 1) / 2)
    sym = sym.clamp(min=0).to(torch.int64).clamp(max=(power - 1).clamp(min=0)[..., None, None])
    # band layout: tiles of a tile row follow each other; a tile of width w takes w rows of 32 words
    offs = torch.cumsum(widths, 1) - widths                                   # offset of each tile within its band
    assert int(offs.max()) < 4096, "a band holds at most 4096 rows of words"
    band_rows = widths.sum(1)
    band_base = torch.cumsum(band_rows, 0) - band_rows
    total_rows = int(band_rows.sum())
    codes = torch.zeros(max(total_rows, 1) * 32 + 32, dtype=torch.int64)
    lane, pair, half = _positions("cpu")
    for tr in range(TR):
        for tc in range(TC):
            wd = int(widths[tr, tc])
            if wd == 0:
                continue
            bit = pair * wd
            shift = bit % 16
            at = (int(band_base[tr]) + int(offs[tr, tc]) + bit // 16) * 32 + lane
            val = sym[tr, tc] << shift                                        # up to 31 bits
            codes.index_put_((at.reshape(-1),), ((val & 0xFFFF) << half).reshape(-1), accumulate=True)
            hi = (val >> 16) & 0xFFFF
            cross = (shift + wd > 16).reshape(-1)
            codes.index_put_(((at + 32).reshape(-1)[cross],), (hi << half).reshape(-1)[cross], accumulate=True)
    tiles_word = (offs & 0xFFF) | (widths << 12) | (scale.view(torch.int16).to(torch.int64) & 0xFFFF) << 16
    to_i32 = lambda x: torch.where(x >= 2 ** 31, x - 2 ** 32, x).to(torch.int32)
    return dict(codes=to_i32(codes), tiles=to_i32(tiles_word), bands=to_i32(band_base),
                row_scale=torch.ones(R), col_scale=torch.ones(C))


def to_group64(fields: dict, dtype=torch.bfloat16, device=None):
    """Re-code a ``fragment`` matrix as the 4-bit group-64 format the decode kernels read."""
    from .decode import quantize_w4
    R, C = fields["tiles"].shape[0] * 32, fields["tiles"].shape[1] * 32
    w = fragment(fields["codes"], fields["tiles"], fields["bands"], fields["row_scale"], fields["col_scale"],
                 torch.arange(R), torch.arange(C), torch.float32)
    return quantize_w4(w.to(device=device or "cuda", dtype=dtype))


class CodedLinear(torch.nn.Module):
    """``y = x W^T`` with ``W`` stored as 4-bit or 8-bit codes and one fp16 scale per group of 64 inputs.

    On bf16 CUDA inputs the codes are dequantised in registers on the way to the tensor cores, never to memory: up to
    8 rows of ``x`` go through the fused decode kernel (weight streaming), more rows through the tcgen05 GEMM with
    dequantising producer warps (``gemm_q``).  Elsewhere (CPU, other dtypes, widths the kernels do not tile) the
    matrix is dequantised and multiplied with PyTorch."""

    def __init__(self, weight: torch.Tensor, bits: int = 4):
        super().__init__()
        from .decode import quantize_w4, quantize_w8
        if bits not in (4, 8):
            raise ValueError("CodedLinear: 4 or 8 bits")
        codes, scales = (quantize_w4 if bits == 4 else quantize_w8)(weight)
        self.bits = bits
        self.register_buffer("codes", codes)
        self.register_buffer("scales", scales)
        self.out_features, self.in_features = weight.shape

    def dense(self) -> torch.Tensor:
        from .decode import dequantize_w4, dequantize_w8
        return (dequantize_w4 if self.bits == 4 else dequantize_w8)(self.codes, self.scales)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.is_cuda and x2.dtype == torch.bfloat16 and x2.shape[0] > 0:
            if x2.shape[0] <= 8 and self.in_features % 512 == 0 and self.out_features % 16 == 0:
                from .decode import decode_linear
                return decode_linear(x2.contiguous(), self.codes, scales=self.scales).reshape(*lead, self.out_features)
            if self.in_features % 64 == 0 and self.out_features % 8 == 0:
                from .gemm import gemm_q
                return gemm_q(x2.contiguous(), self.codes, self.scales).reshape(*lead, self.out_features)
        return torch.nn.functional.linear(x2, self.dense().to(x2.dtype)).reshape(*lead, self.out_features)


# ------------------------------------------------------------------------------------------------ coded matrices
def hadamard_transform(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised fast Walsh-Hadamard transform along the last dimension (a power of two)."""
    n = x.shape[-1]
    if n & (n - 1):
        raise ValueError("the Hadamard transform needs a power-of-two width")
    y, step = x, 1
    while step < n:
        pair = y.reshape(*y.shape[:-1], -1, 2 * step)
        a, b = pair[..., :step], pair[..., step:]
        y = torch.cat((a + b, a - b), -1).reshape(x.shape)
        step *= 2
    return y


class CodedMatrix(torch.nn.Module):
    """A ``fragment``-coded weight matrix with the input transform it was coded under.

    Quantisation error shrinks when the inputs are decorrelated first, so a coded matrix may come with (one of) a
    column order, a dense rotation of the input, or a sign flip followed by a Hadamard transform; ``forward`` applies
    the transform and multiplies by the decoded weights.  ``select`` restricts the matrix to some output rows /
    input columns (tensor-parallel shards).  The fields are those of the reference's ``Matrix``
    (rdma/mesh_code.py:19-64): ``codes, tiles, bands, row_scale, col_scale`` plus optional ``row_order``,
    ``col_order``, ``rotation`` + ``rotation_scale``, ``signs``."""

    def __init__(self, fields: dict, rows=None, columns=None):
        super().__init__()
        self.names = tuple(fields)
        for k, v in fields.items():
            self.register_buffer(k, v)
        R, C = fields["tiles"].shape[0] * 32, fields["tiles"].shape[1] * 32
        row_order = fields.get("row_order", torch.arange(R)).long()
        col_order = fields.get("col_order", torch.arange(C)).long()
        rows = torch.arange(R) if rows is None else torch.as_tensor(rows).long()
        columns = torch.arange(C) if columns is None else torch.as_tensor(columns).long()
        # stored row i holds logical row row_order[i]: find where the wanted logical rows are stored
        self.register_buffer("stored_rows", torch.argsort(row_order)[rows])
        self.register_buffer("input_ids", columns)
        mixes = "rotation" in fields or "signs" in fields
        stored_cols = torch.argsort(col_order)[columns]
        # a transform that mixes the inputs produces all stored columns; otherwise only the selected ones are read
        self.register_buffer("stored_cols", torch.arange(C) if mixes else stored_cols)
        self.shape = (rows.numel(), columns.numel())
        self.width = C

    def select(self, rows=None, columns=None) -> "CodedMatrix":
        return CodedMatrix({k: getattr(self, k) for k in self.names}, rows, columns)

    def transform(self, x: torch.Tensor) -> torch.Tensor:
        if hasattr(self, "rotation"):
            basis = self.rotation.index_select(1, self.input_ids).float() * self.rotation_scale[:, None].float()
            return torch.nn.functional.linear(x, basis.to(x.dtype))
        if hasattr(self, "signs"):
            full = x.new_zeros((*x.shape[:-1], self.width)).index_copy(-1, self.input_ids, x)
            mixed = hadamard_transform(full * self.signs.to(x.dtype)) / self.width ** 0.5
            return mixed.index_select(-1, self.col_order.long()) if hasattr(self, "col_order") else mixed
        return x

    def weight(self, dtype=torch.float32) -> torch.Tensor:
        return fragment(self.codes, self.tiles, self.bands, self.row_scale, self.col_scale, self.stored_rows,
                        self.stored_cols, dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _linear(self.transform(x), self.weight(x.dtype))


def _linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x w^T``: this package's GEMM for bf16 CUDA operands it tiles, PyTorch elsewhere."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 \
            and x.numel() > 0:
        from .gemm import gemm
        return gemm(x.reshape(-1, x.shape[-1]).contiguous(), w.contiguous()).reshape(*x.shape[:-1], w.shape[0])
    return torch.nn.functional.linear(x, w)


class CodedFFN(torch.nn.Module):
    """GeGLU FFN over three coded matrices, restricted to ``count`` hidden units from ``first`` (a tensor-parallel
    share); gate and up share one input transform when they were coded under the same one
    (rdma/mesh_code.py:68-82)."""

    def __init__(self, gate: CodedMatrix, up: CodedMatrix, down: CodedMatrix, first: int = 0, count: int | None = None):
        super().__init__()
        hidden = torch.arange(first, first + (count if count is not None else gate.shape[0] - first))
        self.gate, self.up, self.down = gate.select(rows=hidden), up.select(rows=hidden), down.select(columns=hidden)
        names = ("col_order", "rotation", "rotation_scale", "signs")
        self.shared = all(hasattr(gate, n) == hasattr(up, n) and (not hasattr(gate, n) or torch.equal(getattr(gate, n), getattr(up, n)))
                          for n in names)

    def forward(self, x):
        t = self.gate.transform(x)
        g = _linear(t, self.gate.weight(x.dtype))
        u = _linear(t if self.shared else self.up.transform(x), self.up.weight(x.dtype))
        return self.down(torch.nn.functional.gelu(g, approximate="tanh") * u)


def save_matrices(path, matrices: dict, metadata: dict | None = None) -> None:
    """``{name: fields}`` -> one safetensors file with tensors ``name.field``."""
    from safetensors.torch import save_file
    flat = {f"{n}.{k}": v.contiguous() for n, fields in matrices.items() for k, v in fields.items()}
    save_file(flat, str(path), metadata=metadata or {})


def load_matrices(path) -> dict:
    """The coded matrices of a safetensors file written by :func:`save_matrices` (or by the reference's tooling:
    tensors ``name.codes``, ``name.tiles``, ...; rdma/mesh_code.py:85-101)."""
    from safetensors.torch import load_file
    tensors = load_file(str(path), device="cpu")
    out = {}
    for name in sorted(k[:-6] for k in tensors if k.endswith(".codes")):
        fields = {k[len(name) + 1:]: v for k, v in tensors.items() if k.startswith(name + ".")}
        out[name] = CodedMatrix(fields)
    return out
