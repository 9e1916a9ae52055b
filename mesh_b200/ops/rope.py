"""Rotate-half rotary position embedding (in place) on the hand-written kernel.

Reference model: examples/pl.py:17-28 — cached cos/sin tables and ``rotate_half``.
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p

import torch

from .. import _native


def rope_tables(max_pos: int, head_dim: int, theta: float = 10000.0, device="cuda"):
    """fp32 ``cos, sin`` of shape ``[max_pos, head_dim // 2]``."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def rope_(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False):
    """Rotate ``x[tokens, heads, head_dim]`` in place.  ``x`` may be a column slice of a wider
    matrix (e.g. the q part of a fused qkv output): only the last two dims must be dense."""
    assert x.dtype == torch.bfloat16 and x.is_cuda and x.dim() == 3
    tokens, heads, hd = x.shape
    assert x.stride(2) == 1 and x.stride(1) == hd, "heads must be dense in memory"
    assert positions.dtype == torch.int32 and positions.numel() == tokens
    rc = _native.lib().mesh_rope(c_void_p(x.data_ptr()), c_void_p(positions.data_ptr()), c_void_p(cos.data_ptr()),
                                 c_void_p(sin.data_ptr()), c_int(tokens), c_int(heads), c_int(hd),
                                 c_longlong(x.stride(0)), c_int(int(inverse)),
                                 c_void_p(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "mesh_rope")
    _native.count_launch(1)
    return x


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, cos, sin):
        ctx.save_for_backward(positions, cos, sin)
        y = x.clone()
        rope_(y, positions, cos, sin)
        return y

    @staticmethod
    def backward(ctx, dy):
        positions, cos, sin = ctx.saved_tensors
        dx = dy.clone()
        rope_(dx, positions, cos, sin, inverse=True)
        return dx, None, None, None


def rope(x, positions, cos, sin):
    return _Rope.apply(x, positions, cos, sin)


def rope_ref(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """fp32 PyTorch statement (oracle / CPU path)."""
    xf = x.float()
    half = x.shape[-1] // 2
    c = cos[positions.long()][:, None, :].to(xf.device)
    s = sin[positions.long()][:, None, :].to(xf.device)
    a, b = xf[..., :half], xf[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)
