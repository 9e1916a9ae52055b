"""Decode-time kernels: fused skinny linear layers, split-KV attention, vocabulary-parallel argmax,
and the 4-bit group-64 weight format they read.

Reference: the E2B decode analysis (design/e2b-crossover-2026-09-16.md) and the coded-weight op
``mesh::fragment`` (rdma/mesh_code.py:9-16).  The 4-bit format here is the benchmark's "4-bit group-64
with fp16 scales": ``w ~ (code - 8) * scale[row, k // 64]``; eight codes are packed per 32-bit word
in nibble order ``0,4,1,5,2,6,3,7`` so that the kernel can split pairs with one mask.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint32, c_void_p

import torch

from .. import _native
from ..utils.status import status_block

STORE, GLU, QKV, ALLREDUCE = 0, 1, 2, 3
MAX_RANKS = 8
_NIB = [0, 4, 1, 5, 2, 6, 3, 7]


class _Lin(ctypes.Structure):
    _fields_ = [
        ("x", c_void_p), ("ldx", c_longlong), ("B", c_int), ("K", c_int), ("N", c_int),
        ("norm_w", c_void_p), ("eps", c_float), ("norm_off", c_float),
        ("w", c_void_p), ("scales", c_void_p), ("w4", c_int),
        ("mode", c_int), ("act", c_int), ("up_off", c_int),
        ("out", c_void_p), ("ldo", c_longlong), ("out_f32", c_int),
        ("q_heads", c_int), ("kv_heads", c_int), ("head_dim", c_int),
        ("pos", c_void_p), ("cos_t", c_void_p), ("sin_t", c_void_p),
        ("q_out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("max_seq", c_int),
        ("rank", c_int), ("world", c_int),
        ("ar_recv", c_void_p * MAX_RANKS),
        ("step_ptr", c_void_p), ("calls_per_step", c_uint32), ("call_index", c_uint32),
        ("residual", c_void_p), ("ldr", c_longlong),
        ("status", c_void_p),
        ("next_w", c_void_p), ("next_bytes", ctypes.c_uint64),
    ]


def quantize_w4(w: torch.Tensor, group: int = 64):
    """``w [N, K]`` -> ``(codes uint8 [N, K/2] in the kernel's packing, scales fp16 [N, K/group])``."""
    assert group == 64 and w.dim() == 2 and w.shape[1] % 64 == 0
    N, K = w.shape
    wf = w.float().view(N, K // group, group)
    scale = (wf.abs().amax(-1) / 7.0).clamp_min(1e-8)
    scale = scale.to(torch.float16)
    codes = torch.clamp(torch.round(wf / scale.float()[..., None]) + 8, 0, 15).to(torch.int32).view(N, K // 8, 8)
    word = torch.zeros((N, K // 8), dtype=torch.int64, device=w.device)
    for j in range(8):
        word |= codes[:, :, j].to(torch.int64) << (4 * _NIB[j])
    word = torch.where(word >= (1 << 31), word - (1 << 32), word).to(torch.int32)
    return word.view(torch.uint8).view(N, K // 2).contiguous(), scale.contiguous()


def dequantize_w4(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`quantize_w4` in plain PyTorch (oracle; also the prefill path's weights)."""
    N = codes.shape[0]
    K = codes.shape[1] * 2
    word = codes.contiguous().view(torch.int32).view(N, K // 8).to(torch.int64) & 0xFFFFFFFF
    vals = torch.stack([((word >> (4 * _NIB[j])) & 0xF) for j in range(8)], dim=-1).view(N, K).float() - 8.0
    return (vals.view(N, K // 64, 64) * scales.float()[..., None]).view(N, K).to(torch.bfloat16)


def quantize_w8(w: torch.Tensor, group: int = 64):
    """``w [N, K]`` -> ``(codes uint8 [N, K], scales fp16 [N, K/group])``: ``w ~ (code - 128) * scale[row, k // 64]``,
    codes in the natural order of k (the north star's 8-bit group-quantised variant)."""
    assert group == 64 and w.dim() == 2 and w.shape[1] % 64 == 0
    N, K = w.shape
    wf = w.float().view(N, K // group, group)
    scale = (wf.abs().amax(-1) / 127.0).clamp_min(1e-8).to(torch.float16)
    codes = torch.clamp(torch.round(wf / scale.float()[..., None]) + 128, 1, 255).to(torch.uint8)
    return codes.view(N, K).contiguous(), scale.contiguous()


def dequantize_w8(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    N, K = codes.shape
    return ((codes.float() - 128.0).view(N, K // 64, 64) * scales.float()[..., None]).view(N, K).to(torch.bfloat16)


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t) -> int:
    return 0 if t is None else t.data_ptr()


def decode_linear(x: torch.Tensor, w: torch.Tensor, *, scales: torch.Tensor | None = None, n_rows: int | None = None,
                  norm_w: torch.Tensor | None = None, eps: float = 1e-6, norm_off: float = 0.0,
                  mode: int = STORE, act: str = "gelu_tanh", up_off: int = 0,
                  out: torch.Tensor | None = None, out_f32: bool = False, residual: torch.Tensor | None = None,
                  qkv: dict | None = None, ar: dict | None = None, next_weights: torch.Tensor | None = None) -> torch.Tensor | None:
    """One fused skinny linear layer.  ``x [B<=8, K]`` bf16; ``w`` bf16 ``[rows, K]``, or uint8 codes with
    ``scales`` (``[rows, K/2]``: 4-bit, :func:`quantize_w4`; ``[rows, K]``: 8-bit, :func:`quantize_w8`).

    ``mode``: STORE (``out[b, n]``, optional ``residual`` added) | GLU (``w = [gate; up]``, ``up_off`` = gate rows) |
    QKV (``qkv`` = dict(q_heads, kv_heads, head_dim, pos, cos, sin, q_out, k_cache, v_cache, max_seq)) |
    ALLREDUCE (``ar`` = dict(rank, world, recv_ptrs, step, calls_per_step, call_index); sums the ranks' partial
    outputs, adds ``residual``).  ``next_weights``: the weight matrix of the linear layer that follows in the step; this
    kernel asks for its first ``MESH_DECODE_PREFETCH_MB`` (default 8) megabytes to be brought into L2 while it streams its
    own, so that HBM does not sit idle across the kernel boundary.
    """
    B, K = x.shape
    w4 = 0                                   # weight format: 0 bf16, 1 4-bit codes, 8 8-bit codes
    if scales is not None:
        w4 = 8 if w.shape[1] == K else 1
        if w4 == 1 and w.shape[1] * 2 != K:
            raise ValueError(f"decode_linear: codes of width {w.shape[1]} do not fit K = {K} in 4 or 8 bits")
    rows = w.shape[0]
    d = _Lin()
    d.x, d.ldx, d.B, d.K = x.data_ptr(), x.stride(0), B, K
    d.N = n_rows if n_rows is not None else (rows // 2 if mode == GLU else rows)
    d.norm_w, d.eps, d.norm_off = _p(norm_w), eps, norm_off
    d.w, d.scales, d.w4 = w.data_ptr(), _p(scales), int(w4)
    d.mode, d.act, d.up_off = mode, 0 if act in ("silu", "swiglu") else 1, up_off if mode == GLU and up_off else (rows // 2 if mode == GLU else 0)
    if mode in (STORE, GLU, ALLREDUCE):
        if out is None:
            out = torch.empty((B, d.N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
        d.out, d.ldo, d.out_f32 = out.data_ptr(), out.stride(0), int(out.dtype == torch.float32)
    if residual is not None:
        d.residual, d.ldr = residual.data_ptr(), residual.stride(0)
    if mode == QKV:
        d.q_heads, d.kv_heads, d.head_dim = qkv["q_heads"], qkv["kv_heads"], qkv["head_dim"]
        d.pos, d.cos_t, d.sin_t = qkv["pos"].data_ptr(), qkv["cos"].data_ptr(), qkv["sin"].data_ptr()
        d.q_out, d.k_cache, d.v_cache, d.max_seq = qkv["q_out"].data_ptr(), qkv["k_cache"].data_ptr(), qkv["v_cache"].data_ptr(), qkv["max_seq"]
    d.world = 1
    if mode == ALLREDUCE:
        d.rank, d.world = ar["rank"], ar["world"]
        for r in range(d.world):
            d.ar_recv[r] = ar["recv_ptrs"][r]
        d.step_ptr, d.calls_per_step, d.call_index = _p(ar.get("step")), ar.get("calls_per_step", 1), ar.get("call_index", 0)
    d.status = status_block(x.device).data_ptr()
    if next_weights is not None:
        d.next_w = next_weights.data_ptr()
        import os
        cap = int(float(os.environ.get("MESH_DECODE_PREFETCH_MB", "8")) * (1 << 20))
        d.next_bytes = min(next_weights.numel() * next_weights.element_size(), cap)
    rc = _native.lib().mesh_decode_linear(ctypes.byref(d), _stream())
    _native.check(rc, "mesh_decode_linear")
    _native.count_launch()
    return out


class DecodeAttention:
    """Split-KV attention workspace for a fixed (batch, heads) shape."""

    def __init__(self, B: int, q_heads: int, kv_heads: int, head_dim: int, splits: int = 16, tokens_per_seq: int = 1,
                 device="cuda"):
        self.B, self.T, self.qh, self.kvh, self.hd, self.splits = B, tokens_per_seq, q_heads, kv_heads, head_dim, splits
        L = _native.lib()
        n = L.mesh_decode_attention_scratch_floats(c_int(B * tokens_per_seq), c_int(q_heads), c_int(head_dim), c_int(splits))
        self.scratch = torch.empty(n, dtype=torch.float32, device=device)
        self.counters = torch.zeros(B * tokens_per_seq * kv_heads, dtype=torch.int32, device=device)

    def __call__(self, q, k_cache, v_cache, pos, out, window: int = 0, scale: float | None = None):
        scale = self.hd ** -0.5 if scale is None else scale
        rc = _native.lib().mesh_decode_attention(
            c_void_p(q.data_ptr()), c_void_p(k_cache.data_ptr()), c_void_p(v_cache.data_ptr()), c_void_p(pos.data_ptr()),
            c_void_p(out.data_ptr()), c_void_p(self.scratch.data_ptr()), c_void_p(self.counters.data_ptr()),
            c_int(self.B), c_int(self.T), c_int(self.qh), c_int(self.kvh), c_int(self.hd), c_int(k_cache.shape[-2]),
            c_int(window), c_float(scale), c_int(self.splits), _stream())
        _native.check(rc, "mesh_decode_attention")
        _native.count_launch()
        return out


def decode_argmax(logits: torch.Tensor, tokens_out: torch.Tensor, pos: torch.Tensor | None, vocab_offset: int = 0,
                  rank: int = 0, world: int = 1, xchg_ptrs: list[int] | None = None, step: torch.Tensor | None = None):
    B, V = logits.shape
    arr = (c_void_p * MAX_RANKS)(*([c_void_p(p) for p in (xchg_ptrs or [])] + [c_void_p(0)] * (MAX_RANKS - len(xchg_ptrs or []))))
    rc = _native.lib().mesh_decode_argmax(c_void_p(logits.data_ptr()), c_longlong(logits.stride(0)), c_int(B), c_int(V),
                                          c_int(vocab_offset), c_void_p(tokens_out.data_ptr()), c_void_p(_p(pos)),
                                          c_int(rank), c_int(world), arr, c_void_p(_p(step)),
                                          c_void_p(status_block(logits.device).data_ptr()), _stream())
    _native.check(rc, "mesh_decode_argmax")
    _native.count_launch()
    return tokens_out
