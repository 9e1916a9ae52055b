"""Numerics of a compiled program on a B200: which steps run on this package's kernels.

The reference's compiler owns its numerics: every operator of a placed graph becomes typed records that its own
generated kernels execute (compiler/mesh_compiler/operations.py:7519-7549, ``SOURCES``), attention as one blockwise
operator (:7081-7166), products as one contraction (:1191-1272), norms as one normalisation (:6671-6682).  Here the
executor asks this table before it falls back to the PyTorch operator: on bf16 CUDA operands a product runs on the
tcgen05 GEMM, whole attention on the flash kernel (also when the queries are a sequence shard: the kernel takes the
logical row positions), and the chain of operators an RMS norm is captured as runs as the one RMSNorm kernel (the
chain is found by ``fuse.fuse_norms``).  Everything else, and every operand that is not bf16 on a GPU or that the
kernels do not tile, stays on the PyTorch operator: the program is the same program either way.

``counts`` (``{"own": n, "eager": n}``) is what ``Program.structure()`` reports.
"""
from __future__ import annotations

import os

import torch

aten = torch.ops.aten


def enabled() -> bool:
    return os.environ.get("MESH_COMPILED_KERNELS", "1") != "0"


def _bf16_cuda(*ts) -> bool:
    return all(isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.bfloat16 for t in ts)


def _rowmajor(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.shape[1] and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def mm(a: torch.Tensor, b: torch.Tensor):
    """``a [M, K] @ b [K, N]`` on the tcgen05 GEMM, or ``None`` when the operands do not fit it."""
    if not _bf16_cuda(a, b) or a.dim() != 2 or b.dim() != 2 or a.shape[0] == 0:
        return None
    M, K = a.shape
    N = b.shape[1]
    if K % 8 or N % 8 or K == 0 or N == 0:
        return None
    from ..ops.gemm import gemm
    a_mn = False
    if not _rowmajor(a):
        if _rowmajor(a.t()) and M % 64 == 0:            # a is a transposed view of a stored [K, M] matrix
            a, a_mn = a.t(), True
        else:
            a = a.contiguous()
    if _rowmajor(b.t()):                                  # b is a transposed view of a stored [N, K] matrix (a weight)
        return gemm(a, b.t(), a_mn=a_mn)
    if not _rowmajor(b):
        b = b.contiguous()
    if N % 64:
        return None                                       # an MN-major operand is tiled in 64-column groups
    return gemm(a, b, a_mn=a_mn, b_mn=True)


def attention(q, k, v, *, causal: bool, scale=None, row_positions=None, dropout_p: float = 0.0, mask=None, dropout=None):
    """Whole attention, ``q [B, H, Tq, hd]``, ``k, v [B, Hkv, Tk, hd]`` as the captured operator has them, on the flash
    kernel; ``row_positions``: ``(first, stride)`` of the query rows in the whole sequence when they are a shard.
    ``dropout``: the kernel's dropout description (``ops/attention.py::_set_dropout``) when the operator drops
    probabilities; its mask is a function of logical coordinates, so a cut of the heads or of the sequence changes
    nothing.  ``None`` when the kernel does not take the case (a mask tensor, dropout without a description, a head
    size it has no tiles for)."""
    if mask is not None or (dropout_p and not dropout) or not _bf16_cuda(q, k, v) or q.dim() != 4:
        return None
    B, H, Tq, hd = q.shape
    Hkv, Tk = k.shape[1], k.shape[2]
    if hd not in (64, 128, 256) or H % Hkv or Tq == 0 or Tk == 0:
        return None
    from ..ops.attention import flash_attention
    qt, kt, vt = (t.transpose(1, 2).contiguous() for t in (q, k, v))          # [B, T, H, hd]
    off, stride = (0, 1) if row_positions is None else row_positions
    if causal and row_positions is None and Tq != Tk:
        return None
    out = flash_attention(qt, kt, vt, causal=causal, scale=scale, q_off=off, q_stride=stride,
                          dropout=dropout if dropout_p else None)
    return out.transpose(1, 2)


def rms_norm(x: torch.Tensor, w, eps: float):
    """``x * rsqrt(mean(x^2, -1) + eps) [* w]`` on the RMSNorm kernel, or ``None``."""
    if not _bf16_cuda(x) or x.shape[-1] % 8 or x.shape[-1] > 16384 or x.numel() == 0:
        return None
    if w is not None and not (_bf16_cuda(w) and w.dim() == 1 and w.shape[0] == x.shape[-1]):
        return None
    from ..ops.norm import rmsnorm_fwd
    if w is None:
        w = torch.ones(x.shape[-1], dtype=torch.bfloat16, device=x.device)
    y, _, _ = rmsnorm_fwd(x.contiguous(), w.contiguous(), eps)
    return y


class Counter:
    def __init__(self):
        self.own, self.eager = 0, 0

    def as_dict(self) -> dict:
        return {"own": self.own, "eager": self.eager}
