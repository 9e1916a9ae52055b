"""Source formulations of dense linear-algebra operators, as a decomposition table for the capture stage.

The reference expands numerics that have no device routine into the nodes of a formulation made of operators the
rest of the compiler can place (compiler/mesh_compiler/decompose.py:86-170: ``matrix_exp`` by scaling and squaring,
``pinv`` / ``svd`` / ``lstsq`` / ``eigh`` off the CPU through a QDWH polar decomposition, operations.py:2370-2470).
The reason is a different one on a B200 - cuSOLVER has these routines - but the effect is the one wanted: after the
expansion the work is matrix products (tensor cores), Cholesky factors, triangular solves and pointwise arithmetic,
every one of which has a partition rule, so a batch of factorizations is cut over processors like any other batch
and a single large one is cut through its products.

    scheduled = compile_module(module, args, processors, placement, decompositions=decompose.table())

Formulations (all with static shapes and a fixed operation count, so they export):

* :func:`matrix_exp`   - Pade-13 approximant with scaling and squaring (Higham 2005); the number of squarings is data
  dependent, so ``max_squarings`` squarings are emitted and the unused ones select their input.
* :func:`polar`        - QDWH, the dynamically weighted Halley iteration (Nakatsukasa, Bai, Gygi 2010), started from the
  lower bound ``eps`` on the smallest singular value, which makes the weights compile-time constants; the first
  iterations (large weights) use the stacked-QR form, the later ones the Cholesky form.
* :func:`eigh`         - cyclic Jacobi with the round-robin ordering: each round rotates n/2 disjoint pairs at once,
  written as slices, flips and concatenations of rows and columns; ``sweeps`` is fixed.
* :func:`svd`          - polar decomposition, then :func:`eigh` of the symmetric factor.
* :func:`pinv`, :func:`lstsq` - through :func:`svd` (minimum-norm solution, rank from a relative threshold).
"""
from __future__ import annotations

import math

import torch

aten = torch.ops.aten

_PADE13 = (64764752532480000., 32382376266240000., 7771770303897600., 1187353796428800., 129060195264000.,
           10559470104000., 670442572800., 33522128640., 1323241920., 40840800., 960960., 16380., 182., 1.)
_THETA13 = 5.371920351148152


def _eye_like(a: torch.Tensor) -> torch.Tensor:
    n = a.shape[-1]
    return torch.eye(n, dtype=a.dtype, device=a.device).expand(a.shape[:-2] + (n, n))


def matrix_exp(a: torch.Tensor, max_squarings: int = 16) -> torch.Tensor:
    """``exp(a)`` for square matrices ``[..., n, n]``."""
    if a.shape[-1] != a.shape[-2]:
        raise ValueError("matrix_exp needs square matrices")
    if a.numel() == 0:
        return a.clone()
    work = a.to(torch.float32) if a.dtype in (torch.float16, torch.bfloat16) else a
    norm = work.abs().sum(-2).amax(-1)                                            # 1-norm
    s = torch.ceil(torch.log2(torch.clamp(norm / _THETA13, min=1.0))).clamp(max=float(max_squarings))
    x = work * torch.exp2(-s)[..., None, None]
    eye = _eye_like(x)
    b = _PADE13
    x2 = x @ x
    x4 = x2 @ x2
    x6 = x4 @ x2
    u = x @ (x6 @ (b[13] * x6 + b[11] * x4 + b[9] * x2) + b[7] * x6 + b[5] * x4 + b[3] * x2 + b[1] * eye)
    v = x6 @ (b[12] * x6 + b[10] * x4 + b[8] * x2) + b[6] * x6 + b[4] * x4 + b[2] * x2 + b[0] * eye
    r = torch.linalg.solve(v - u, v + u)
    for i in range(max_squarings):
        r = torch.where((s > i)[..., None, None], r @ r, r)
    return r.to(a.dtype)


def _halley_weights(eps: float, max_iterations: int) -> list[tuple[float, float, float]]:
    """The weights ``(a, b, c)`` of each QDWH iteration when the smallest singular value is only known to be >= eps."""
    out, l = [], float(eps)
    while abs(1.0 - l) > 10 * eps and len(out) < max_iterations:
        l2 = l * l
        dd = (4.0 * (1.0 - l2) / (l2 * l2)) ** (1.0 / 3.0)
        sq = math.sqrt(1.0 + dd)
        a = sq + 0.5 * math.sqrt(8.0 - 4.0 * dd + 8.0 * (2.0 - l2) / (l2 * sq))
        b = (a - 1.0) ** 2 / 4.0
        c = a + b - 1.0
        l = l * (a + b * l2) / (1.0 + c * l2)
        out.append((a, b, c))
    return out + [(3.0, 1.0, 3.0)]                       # one plain Halley step: cubic convergence from |1 - l| ~ eps


def polar(a: torch.Tensor, max_iterations: int = 10):
    """Polar decomposition ``a = u @ h`` of ``[..., m, n]`` with ``m >= n``: ``u`` has orthonormal columns, ``h`` is
    symmetric positive semi-definite."""
    m, n = a.shape[-2:]
    if m < n:
        raise ValueError("polar needs at least as many rows as columns; pass the transpose")
    work = a.to(torch.float32) if a.dtype in (torch.float16, torch.bfloat16) else a
    eps = torch.finfo(work.dtype).eps
    alpha = torch.sqrt(work.abs().sum(-2).amax(-1) * work.abs().sum(-1).amax(-1))          # >= the 2-norm
    alpha = torch.where(alpha > 0, alpha, torch.ones_like(alpha))
    x = work / alpha[..., None, None]
    eye = torch.eye(n, dtype=work.dtype, device=work.device).expand(work.shape[:-2] + (n, n))
    for wa, wb, wc in _halley_weights(eps, max_iterations):
        if wc > 100.0:
            # [sqrt(c) x; I] = [q1; q2] r  ->  x (I + c x^T x)^-1 = q1 q2^T / sqrt(c), without forming the Gram matrix
            q, _ = torch.linalg.qr(torch.cat([math.sqrt(wc) * x, eye], -2))
            x = (wb / wc) * x + ((wa - wb / wc) / math.sqrt(wc)) * (q[..., :m, :] @ q[..., m:, :].mT)
        else:
            z = eye + wc * (x.mT @ x)
            low = torch.linalg.cholesky(z)
            y = torch.linalg.solve_triangular(low, x.mT, upper=False)
            y = torch.linalg.solve_triangular(low.mT, y, upper=True)                      # (I + c x^T x)^-1 x^T
            x = (wb / wc) * x + (wa - wb / wc) * y.mT
    h = x.mT @ work
    h = 0.5 * (h + h.mT)
    return x.to(a.dtype), h.to(a.dtype)


def _shuffled(x: torch.Tensor, dim: int) -> torch.Tensor:
    """The round-robin move along ``dim``: position 0 stays, the last entry comes second, the rest shift by one."""
    last = x.shape[dim]
    return torch.cat([x.narrow(dim, 0, 1), x.narrow(dim, last - 1, 1), x.narrow(dim, 1, last - 2)], dim)


def eigh(a: torch.Tensor, sweeps: int | None = None):
    """Eigenvalues (ascending) and eigenvectors of symmetric ``[..., n, n]`` by cyclic Jacobi rotations.

    Every round rotates the ``n / 2`` disjoint pairs (i, n - 1 - i) of the current ordering at once, then rows and
    columns move one place round-robin, so that ``n - 1`` rounds meet every pair; the rounds are slices, flips and
    concatenations only (no index tensors), which keeps the formulation a graph of plain operators."""
    n = a.shape[-1]
    if a.shape[-2] != n:
        raise ValueError("eigh needs square matrices")
    work = a.to(torch.float32) if a.dtype in (torch.float16, torch.bfloat16) else a
    if n <= 1:
        return work.diagonal(dim1=-2, dim2=-1).to(a.dtype), torch.ones_like(a)
    if sweeps is None:
        sweeps = (8 if work.dtype == torch.float32 else 12) + (2 if n > 64 else 0)
    work = 0.5 * (work + work.mT)
    odd = n % 2
    if odd:                                               # a decoupled extra row and column: every rotation with it is the identity
        work = torch.nn.functional.pad(work, (0, 1, 0, 1))
    size, half = n + odd, (n + odd) // 2
    vec = torch.eye(size, dtype=work.dtype, device=work.device).expand(work.shape[:-2] + (size, size))
    one = torch.ones((), dtype=work.dtype, device=work.device)
    ring = list(range(size))                              # which original index sits at each position
    for _ in range(sweeps * (size - 1)):
        diag = work.diagonal(dim1=-2, dim2=-1)
        app, aqq = diag[..., :half], diag[..., half:].flip(-1)
        apq = work.flip(-1).diagonal(dim1=-2, dim2=-1)[..., :half]
        flat = apq == 0
        theta = (aqq - app) / (2 * torch.where(flat, one, apq))
        t = torch.where(theta >= 0, one, -one) / (theta.abs() + torch.sqrt(theta * theta + 1))
        t = torch.where(flat, torch.zeros_like(t), t)
        c = torch.rsqrt(t * t + 1)
        s = t * c
        cr, sr = c[..., :, None], s[..., :, None]
        top, bottom = work[..., :half, :], work[..., half:, :].flip(-2)
        work = torch.cat([cr * top - sr * bottom, (sr * top + cr * bottom).flip(-2)], -2)
        cc, sc = c[..., None, :], s[..., None, :]
        left, right = work[..., :, :half], work[..., :, half:].flip(-1)
        work = torch.cat([cc * left - sc * right, (sc * left + cc * right).flip(-1)], -1)
        left, right = vec[..., :, :half], vec[..., :, half:].flip(-1)
        vec = torch.cat([cc * left - sc * right, (sc * left + cc * right).flip(-1)], -1)
        if size > 2:
            work = _shuffled(_shuffled(work, -2), -1)
            vec = _shuffled(vec, -1)
            ring = [ring[0], ring[-1]] + ring[1:-1]
    values = work.diagonal(dim1=-2, dim2=-1)
    if odd:
        at = ring.index(n)                                # where the extra index ended up
        values = torch.cat([values[..., :at], values[..., at + 1:]], -1)
        vec = torch.cat([vec[..., :n, :at], vec[..., :n, at + 1:]], -1)
    values, at = torch.sort(values, dim=-1)
    vec = torch.gather(vec, -1, at[..., None, :].expand(vec.shape))
    return values.to(a.dtype), vec.to(a.dtype)


def svd(a: torch.Tensor, max_iterations: int = 10, sweeps: int | None = None):
    """Reduced singular value decomposition ``a = u @ diag(s) @ vh`` (``s`` descending).  Columns of ``u`` that belong
    to singular values of zero are zero, not an orthonormal completion."""
    m, n = a.shape[-2:]
    if m < n:
        u, s, vh = svd(a.mT, max_iterations, sweeps)
        return vh.mT, s, u.mT
    up, h = polar(a, max_iterations)
    w, v = eigh(h, sweeps)
    w, v = w.flip(-1), v.flip(-1)
    return up @ v, w.clamp(min=0), v.mT


def pinv(a: torch.Tensor, rtol: float | None = None, max_iterations: int = 10, sweeps: int | None = None):
    """Moore-Penrose inverse: singular values up to ``rtol`` times the largest count as zero."""
    u, s, vh = svd(a, max_iterations, sweeps)
    if rtol is None:
        dt = torch.float32 if a.dtype in (torch.float16, torch.bfloat16) else a.dtype
        rtol = max(a.shape[-2:]) * torch.finfo(dt).eps
    keep = s > rtol * s.amax(-1, keepdim=True)
    inv = torch.where(keep, 1.0 / torch.where(keep, s, torch.ones_like(s)), torch.zeros_like(s))
    return (vh.mT * inv[..., None, :]) @ u.mT


def lstsq(a: torch.Tensor, b: torch.Tensor, rtol: float | None = None):
    """The minimum-norm ``x`` that minimises ``|a x - b|``.  (``torch.linalg.lstsq`` itself cannot be captured: its
    outputs have data-dependent shapes; call this in the module instead.)"""
    return pinv(a, rtol) @ b


def _eigh_rule(a, UPLO="L", compute_v=True):
    tri = torch.tril(a) + torch.tril(a, -1).mT if UPLO.upper() == "L" else torch.triu(a) + torch.triu(a, 1).mT
    values, vectors = eigh(tri)
    return values, (vectors if compute_v else a.new_empty((0,)))


def _svd_rule(a, full_matrices=False, compute_uv=True, *, driver=None):
    if full_matrices and a.shape[-1] != a.shape[-2]:
        raise NotImplementedError("only the reduced singular value decomposition has a source formulation")
    u, s, vh = svd(a)
    if not compute_uv:
        return a.new_empty((0,)), s, a.new_empty((0,))
    return u, s, vh


def _pinv_rule(a, *, atol=None, rtol=None, hermitian=False):
    if atol is not None:
        raise NotImplementedError("pinv with an absolute tolerance tensor has no source formulation")
    if rtol is not None:
        u, s, vh = svd(a)
        keep = s > rtol[..., None] * s.amax(-1, keepdim=True)
        inv = torch.where(keep, 1.0 / torch.where(keep, s, torch.ones_like(s)), torch.zeros_like(s))
        return (vh.mT * inv[..., None, :]) @ u.mT
    return pinv(a)


def var_mean(x: torch.Tensor, dim=None, *, correction=None, keepdim: bool = False):
    """Variance and mean through sums only, so that a reduction over a cut dimension becomes partial sums and one
    all-reduce (the two-pass form: the mean first, then the mean of squared differences)."""
    dims = list(range(x.ndim)) if dim is None else [d % x.ndim for d in ([dim] if isinstance(dim, int) else dim)]
    count = math.prod(x.shape[d] for d in dims)
    c = 1 if correction is None else correction
    mean = x.mean(dims, keepdim=True)
    diff = x - mean
    var = (diff * diff).sum(dims, keepdim=keepdim) / max(count - c, 0)
    return var, (mean if keepdim else mean.squeeze(dims))


def norms(base: dict | None = None) -> dict:
    """Training-mode batch norm (forward and backward) as means, sums and pointwise arithmetic.  Under a batch cut the
    statistics are then those of the whole batch - what the single-process module computes - at the price of two small
    all-reduces, instead of the operator gathering its input."""
    out = dict(base if base is not None else torch.export.default_decompositions())
    out.update(torch._decomp.get_decompositions([aten._native_batch_norm_legit_functional, aten._native_batch_norm_legit,
                                                 aten.native_batch_norm, aten.native_batch_norm_backward]))
    out[aten.var_mean.correction] = var_mean
    return out


def table(max_squarings: int = 16, base: dict | None = None, keep_attention: bool = True, batch_norm: bool = False) -> dict:
    """The capture stage's decomposition table with the formulations of this module added.

    ``base``: the table to extend (default: ``torch.export.default_decompositions()``); ``keep_attention`` leaves
    ``scaled_dot_product_attention`` whole, as the capture stage does for inference graphs (pass ``False`` for a joint
    forward+backward capture); ``batch_norm`` adds :func:`norms`."""
    out = dict(base if base is not None else torch.export.default_decompositions())
    if batch_norm:
        out = norms(out)
    if keep_attention:
        out.pop(aten.scaled_dot_product_attention.default, None)
    out[aten.linalg_matrix_exp.default] = lambda a: matrix_exp(a, max_squarings)
    out[aten._linalg_eigh.default] = _eigh_rule
    out[aten._linalg_svd.default] = _svd_rule
    out[aten.linalg_pinv.atol_rtol_tensor] = _pinv_rule
    return out


EXPANDED = (aten.linalg_matrix_exp.default, aten._linalg_eigh.default, aten._linalg_svd.default,
            aten.linalg_pinv.atol_rtol_tensor)
