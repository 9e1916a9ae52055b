"""RMSNorm (optionally fused with the residual add) on the hand-written sm_100a kernel.

Reference semantics: the ``rms`` member of ``NORMS`` (compiler/mesh_compiler/operations.py:6671-6682)
and the RMSNorm modules of examples/parallel.py:28-36.  ``weight_offset=1.0`` gives the Gemma form
``x * rstd * (1 + w)``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from .. import _native


def _s() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, residual: torch.Tensor | None = None,
                weight_offset: float = 0.0, need_rstd: bool = False, out: torch.Tensor | None = None):
    """Returns ``(y, new_residual or None, rstd or None)``; when ``residual`` is given the sum
    ``x + residual`` is written to ``new_residual`` and normalised."""
    assert x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols
    y = torch.empty_like(x) if out is None else out
    res_out = torch.empty_like(x) if residual is not None else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if need_rstd else None
    L = _native.lib()
    rc = L.mesh_rmsnorm_fwd(_p(x), _p(residual), _p(w), _p(y), _p(res_out), _p(rstd), c_int(rows), c_int(cols),
                            c_float(eps), c_float(weight_offset), _s())
    _native.check(rc, "mesh_rmsnorm_fwd")
    _native.count_launch(1)
    return y, res_out, rstd


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor, weight_offset: float = 0.0):
    cols = x.shape[-1]
    rows = x.numel() // cols
    L = _native.lib()
    blocks = L.mesh_rmsnorm_bwd_blocks(c_int(rows))
    dx = torch.empty_like(x)
    dw = torch.empty(cols, dtype=torch.float32, device=x.device)
    partial = torch.empty((blocks, cols), dtype=torch.float32, device=x.device)
    rc = L.mesh_rmsnorm_bwd(_p(dy.contiguous()), _p(x), _p(w), _p(rstd), _p(dx), _p(dw), _p(partial), c_int(blocks),
                            c_int(rows), c_int(cols), c_float(weight_offset), _s())
    _native.check(rc, "mesh_rmsnorm_bwd")
    _native.count_launch(2)
    return dx, dw


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, weight_offset):
        xc = x.contiguous()
        y, _, rstd = rmsnorm_fwd(xc, w, eps, None, weight_offset, need_rstd=True)
        ctx.save_for_backward(xc, w, rstd)
        ctx.weight_offset = weight_offset
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx, dw = rmsnorm_bwd(dy, x, w, rstd, ctx.weight_offset)
        return dx, dw.to(w.dtype), None, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, weight_offset: float = 0.0) -> torch.Tensor:
    return _RMSNorm.apply(x, w, eps, weight_offset)


def rmsnorm_ref(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, weight_offset: float = 0.0) -> torch.Tensor:
    """Plain PyTorch fp32 statement of the same op (oracle; also the CPU path)."""
    xf = x.float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * r * (w.float() + weight_offset)).to(x.dtype)
