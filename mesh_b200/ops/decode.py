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


class _Op(ctypes.Structure):
    """``MeshDecodeOp``: one operation of a step program (``csrc/ops/decode_api.h``)."""
    _fields_ = [
        ("kind", c_int), ("lin", _Lin),
        ("q", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("pos", c_void_p), ("att_out", c_void_p),
        ("scratch", c_void_p), ("counters", c_void_p),
        ("B", c_int), ("q_heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("max_seq", c_int), ("window", c_int),
        ("scale", c_float), ("splits", c_int),
        ("table", c_void_p), ("tok", c_void_p), ("x", c_void_p), ("d_model", c_int),
        ("logits", c_void_p), ("ldl", c_longlong), ("vocab_local", c_int), ("vocab_offset", c_int),
        ("tokens_out", c_void_p), ("pos_inc", c_void_p), ("rank", c_int), ("world", c_int),
        ("xchg", c_void_p * MAX_RANKS), ("step", c_void_p), ("part_v", c_void_p), ("part_i", c_void_p),
        ("status", c_void_p),
    ]


class _StepPlan(ctypes.Structure):
    _fields_ = [("n_dev", c_int), ("grid", c_int), ("smem", c_int), ("ring_off", c_int), ("slot_bytes", c_int),
                ("n_stages", c_int)]


OP_EMBED, OP_LINEAR, OP_ATTENTION, OP_ARGMAX = 0, 1, 2, 3
_recording: list | None = None           # operations of the step being recorded (``record_step``)


class DecodeStep:
    """A decode step as one cooperative kernel.  Record the step's calls once::

        with record_step(device) as step:
            model._decode_step()          # decode_embed / decode_linear / DecodeAttention / decode_argmax calls
        step.run()                        # every later token: one launch

    Inside the block the calls launch nothing; they describe the operations, which ``run`` executes in that order with a
    grid barrier between them, one CTA per SM, the weights of all layers streamed through shared memory by a warp that
    does not wait at the barriers.  The tensors the calls named are kept alive by the step and must keep their addresses."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.ops: list = []
        self.keep: list = []
        self.dev_ops = None
        self.n_dev = self.grid = self.smem = 0

    def __enter__(self):
        global _recording
        if _recording is not None:
            raise RuntimeError("a decode step is already being recorded")
        _recording = self.ops
        return self

    def __exit__(self, et, ev, tb):
        global _recording
        _recording = None
        if et is None:
            self._prepare()
        return False

    def _prepare(self):
        L = _native.lib()
        n = len(self.ops)
        if n == 0:
            raise RuntimeError("record_step: the block made no decode call")
        arr = (_Op * n)()
        max_grid = int(L.mesh_decode_step_max_grid())
        for i, (op, keep) in enumerate(self.ops):
            if op.kind == OP_ARGMAX:
                pv = torch.empty(op.B * max_grid, dtype=torch.float32, device=self.device)
                pi = torch.empty(op.B * max_grid, dtype=torch.int32, device=self.device)
                op.part_v, op.part_i = pv.data_ptr(), pi.data_ptr()
                self.keep += [pv, pi]
            ctypes.memmove(ctypes.byref(arr, i * ctypes.sizeof(_Op)), ctypes.byref(op), ctypes.sizeof(_Op))
            self.keep.append(keep)
        L.mesh_decode_step_bytes.restype = ctypes.c_size_t
        nbytes = int(L.mesh_decode_step_bytes(c_int(n)))
        self.dev_ops = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.barrier = torch.zeros(2, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        self.plan = _StepPlan()
        rc = L.mesh_decode_step_prepare(arr, c_int(n), c_void_p(self.dev_ops.data_ptr()), ctypes.c_size_t(nbytes),
                                        ctypes.byref(self.plan))
        _native.check(rc, "mesh_decode_step_prepare")
        self.n_dev, self.grid, self.smem = self.plan.n_dev, self.plan.grid, self.plan.smem
        self.status = status_block(self.device)

    def run(self, trace: torch.Tensor | None = None):
        """One step.  ``trace``: an int64 tensor of ``2 * 3 * n_dev`` words on the device; the first and the last CTA
        write {start, end of own share, nanoseconds waited} per operation (see :meth:`timeline`)."""
        rc = _native.lib().mesh_decode_step_run(c_void_p(self.dev_ops.data_ptr()), ctypes.byref(self.plan),
                                                c_void_p(self.barrier.data_ptr()), c_void_p(self.status.data_ptr()),
                                                c_void_p(_p(trace)), _stream())
        _native.check(rc, "mesh_decode_step_run")
        _native.count_launch()

    def kinds(self) -> list[str]:
        """Name of every device operation of the step, in order."""
        names = []
        for op, _ in self.ops:
            if op.kind == OP_LINEAR:
                names.append(("linear", "glu", "qkv", "linear+allreduce")[op.lin.mode] + f" {op.lin.N}x{op.lin.K}")
            elif op.kind == OP_ATTENTION:
                names.append("attention")
            elif op.kind == OP_EMBED:
                names.append("embed")
            else:
                names += ["argmax slices", "argmax merge"]
        return names

    def timeline(self) -> list[dict]:
        """Runs one step with the trace on and returns, per operation, microseconds from the step's start to the
        operation's start and end on the first CTA, and the microseconds the first and the last CTA waited at the
        barrier before it."""
        t = torch.zeros(2 * 3 * self.n_dev, dtype=torch.int64, device=self.device)
        self.run(trace=t)
        torch.cuda.synchronize(self.device)
        v = t.cpu().view(2, self.n_dev, 3)
        t0 = int(v[0, 0, 0])
        return [{"op": name, "start_us": (int(v[0, i, 0]) - t0) / 1e3, "end_us": (int(v[0, i, 1]) - t0) / 1e3,
                 "waited_us": int(v[0, i, 2]) / 1e3, "last_cta_end_us": (int(v[1, i, 1]) - t0) / 1e3,
                 "last_cta_waited_us": int(v[1, i, 2]) / 1e3}
                for i, name in enumerate(self.kinds())]


def record_step(device="cuda") -> DecodeStep:
    return DecodeStep(device)


def decode_embed(table: torch.Tensor, tok: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[b, :] = table[tok[b], :]`` (bf16 rows): the step's first operation."""
    if _recording is not None:
        op = _Op()
        op.kind = OP_EMBED
        op.table, op.tok, op.x, op.B, op.d_model = table.data_ptr(), tok.data_ptr(), out.data_ptr(), tok.shape[0], table.shape[1]
        if not (out.is_contiguous() and table.is_contiguous() and table.dtype == torch.bfloat16):
            raise ValueError("decode_embed: contiguous bf16 table and output")
        _recording.append((op, (table, tok, out)))
        return out
    return torch.index_select(table, 0, tok, out=out)


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
    if _recording is not None:
        op = _Op()
        op.kind = OP_LINEAR
        op.lin = d
        _recording.append((op, (x, w, scales, norm_w, out, residual, qkv, ar)))
        return out
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
        if _recording is not None:
            if self.T != 1:
                raise ValueError("a recorded step decodes one token per sequence")
            op = _Op()
            op.kind = OP_ATTENTION
            op.q, op.k_cache, op.v_cache, op.pos, op.att_out = (q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                                                pos.data_ptr(), out.data_ptr())
            op.scratch, op.counters = self.scratch.data_ptr(), self.counters.data_ptr()
            op.B, op.q_heads, op.kv_heads, op.head_dim, op.max_seq = self.B, self.qh, self.kvh, self.hd, k_cache.shape[-2]
            op.window, op.scale, op.splits = window, scale, self.splits
            _recording.append((op, (q, k_cache, v_cache, pos, out, self)))
            return out
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
    if _recording is not None:
        op = _Op()
        op.kind = OP_ARGMAX
        op.logits, op.ldl, op.B, op.vocab_local, op.vocab_offset = logits.data_ptr(), logits.stride(0), B, V, vocab_offset
        op.tokens_out, op.pos_inc, op.rank, op.world = tokens_out.data_ptr(), _p(pos), rank, world
        for r, ptr in enumerate(xchg_ptrs or []):
            op.xchg[r] = ptr
        op.step, op.status = _p(step), status_block(logits.device).data_ptr()
        _recording.append((op, (logits, tokens_out, pos, step)))
        return tokens_out
    arr = (c_void_p * MAX_RANKS)(*([c_void_p(p) for p in (xchg_ptrs or [])] + [c_void_p(0)] * (MAX_RANKS - len(xchg_ptrs or []))))
    rc = _native.lib().mesh_decode_argmax(c_void_p(logits.data_ptr()), c_longlong(logits.stride(0)), c_int(B), c_int(V),
                                          c_int(vocab_offset), c_void_p(tokens_out.data_ptr()), c_void_p(_p(pos)),
                                          c_int(rank), c_int(world), arr, c_void_p(_p(step)),
                                          c_void_p(status_block(logits.device).data_ptr()), _stream())
    _native.check(rc, "mesh_decode_argmax")
    _native.count_launch()
    return tokens_out
