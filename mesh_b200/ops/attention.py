"""Attention on the hand-written kernels: flash forward (tcgen05), partial-result merging, ring attention.

Reference semantics: blockwise online-softmax attention with ring rotation over context-parallel ranks, striped
logical positions, GQA (compiler/mesh_compiler/operations.py:7081-7166; placement ``units="striped"``,
placement.py:57-69).
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint32, c_uint64, c_void_p

import torch

from .. import _native
from ..utils.status import status_block


class _Flash(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p), ("lse", c_void_p),
                ("ldq", c_longlong), ("ldk", c_longlong), ("ldv", c_longlong), ("ldo", c_longlong),
                ("q_cols", c_int), ("k_cols", c_int), ("v_cols", c_int), ("q_col0", c_int), ("k_col0", c_int), ("v_col0", c_int),
                ("B", c_int), ("H", c_int), ("Hkv", c_int), ("Tq", c_int), ("Tk", c_int), ("head_dim", c_int),
                ("causal", c_int), ("window", c_int), ("q_off", c_int), ("q_stride", c_int), ("k_off", c_int),
                ("k_stride", c_int), ("scale", c_float), ("status", c_void_p),
                ("dropout_p", c_float), ("seed", c_uint64), ("site", c_uint32), ("execution", c_uint32),
                ("head_off", c_int), ("heads_total", c_int)]


def _view2d(t: torch.Tensor):
    """``t [B, T, H, hd]`` (possibly a column slice of a wider fused matrix) -> (base ptr of the row-major parent, ld, col0)."""
    B, T, H, hd = t.shape
    assert t.stride(3) == 1 and t.stride(2) == hd and (B == 1 or t.stride(0) == T * t.stride(1)), \
        "need [B, T, H, hd] with dense heads and batch entries back to back"
    return t.data_ptr(), t.stride(1), H * hd


def _set_dropout(a, dropout) -> None:
    """``dropout``: ``None`` or a dict ``p, seed, site=0, execution=0, head_off=0, heads_total=None``.  The keep mask
    is a function of the logical coordinates (batch, head_off + head of heads_total, query position, key position):
    every shard of the heads or of the sequence drops what one device would (``ops/philox.py::attention_keep_mask``)."""
    if not dropout or not dropout.get("p"):
        return
    a.dropout_p = float(dropout["p"])
    a.seed = int(dropout.get("seed", 0)) & 0xFFFFFFFFFFFFFFFF
    a.site, a.execution = int(dropout.get("site", 0)) & 0xFFFFFFFF, int(dropout.get("execution", 0)) & 0xFFFFFFFF
    a.head_off = int(dropout.get("head_off", 0))
    a.heads_total = int(dropout.get("heads_total") or 0)


def flash_attention(q, k, v, *, causal=True, window=0, scale=None, q_off=0, q_stride=1, k_off=0, k_stride=1,
                    need_lse=False, out=None, dropout=None):
    """``q [B, Tq, H, hd]``, ``k, v [B, Tk, Hkv, hd]`` bf16 -> ``out [B, Tq, H, hd]`` (and ``lse [B, H, Tq]``).
    ``dropout``: see :func:`_set_dropout` (dropout of the attention probabilities, inside the kernel)."""
    B, Tq, H, hd = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    scale = hd ** -0.5 if scale is None else scale
    if out is None:
        out = torch.empty((B, Tq, H, hd), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device) if need_lse else None
    a = _Flash()
    a.q, a.ldq, a.q_cols = _view2d(q)
    a.k, a.ldk, a.k_cols = _view2d(k)
    a.v, a.ldv, a.v_cols = _view2d(v)
    a.out, a.ldo = out.data_ptr(), out.stride(1)
    a.lse = 0 if lse is None else lse.data_ptr()
    a.B, a.H, a.Hkv, a.Tq, a.Tk, a.head_dim = B, H, Hkv, Tq, Tk, hd
    a.causal, a.window = int(causal), int(window)
    a.q_off, a.q_stride, a.k_off, a.k_stride = q_off, q_stride, k_off, k_stride
    a.scale = scale
    a.status = status_block(q.device).data_ptr()
    _set_dropout(a, dropout)
    rc = _native.lib().mesh_flash_attention_fwd(ctypes.byref(a), c_void_p(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "mesh_flash_attention_fwd")
    _native.count_launch()
    return (out, lse) if need_lse else out


def merge_partials(o1, lse1, o2, lse2):
    """Merge two attention results over disjoint key sets: ``o [B, T, H, hd]``, ``lse [B, H, T]``."""
    m = torch.maximum(lse1, lse2)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1, w2 = torch.exp(lse1 - m_safe), torch.exp(lse2 - m_safe)
    tot = w1 + w2
    inv = torch.where(tot > 0, 1.0 / tot, torch.zeros_like(tot))
    a1 = (w1 * inv).transpose(1, 2).unsqueeze(-1)
    a2 = (w2 * inv).transpose(1, 2).unsqueeze(-1)
    o = (o1.float() * a1 + o2.float() * a2).to(o1.dtype)
    return o, m_safe + torch.log(torch.where(tot > 0, tot, torch.ones_like(tot))) + torch.where(tot > 0, 0.0, float("-inf"))


def ring_attention(q, k, v, comm, *, causal=True, striped=False, scale=None, overlap: bool | None = None):
    """Context-parallel attention: every rank holds a sequence shard of q, k, v (contiguous blocks, or striped
    tokens ``r, r+P, ...``); the KV shards travel around the ring while each rank attends its queries to the chunk
    it currently holds, starting with its own (the reference rotates the key loop to start at the rank's own block,
    operations.py:7089-7094), and partial results are merged by their log-sum-exp.  Chunks that the causal mask
    hides completely are skipped.

    ``overlap`` (default: environment ``MESH_RING_OVERLAP=1``): pass the next chunk on a side stream, so that the
    transfer runs under the attention of the current chunk instead of before it."""
    import os
    if overlap is None:
        overlap = os.environ.get("MESH_RING_OVERLAP", "0") == "1"
    P, r = comm.world, comm.rank
    B, T, H, hd = q.shape
    kv = torch.stack([k, v]).contiguous()
    o, lse = None, None
    main = torch.cuda.current_stream(q.device) if q.is_cuda else None
    side = _ring_stream(q.device) if (overlap and q.is_cuda and P > 1) else None
    ring = [(j, (j + 1) % P) for j in range(P)]
    for step in range(P):
        src = (r - step) % P                                  # whose KV chunk we hold at this step
        if striped:
            q_off, q_stride, k_off, k_stride = r, P, src, P
        else:
            q_off, q_stride, k_off, k_stride = r * T, 1, src * T, 1
        visible = (not causal) or striped or src <= r
        nxt = None
        if step + 1 < P:                                      # pass the chunk on while we compute
            nxt = torch.empty_like(kv)
            if side is not None:
                side.wait_stream(main)                        # kv is complete; nxt is allocated
                with torch.cuda.stream(side):
                    comm.permute(nxt, kv, ring)
                kv.record_stream(side)
                nxt.record_stream(side)
            else:
                comm.permute(nxt, kv, ring)
        if visible:
            oi, li = flash_attention(q, kv[0], kv[1], causal=causal, scale=scale, q_off=q_off, q_stride=q_stride,
                                     k_off=k_off, k_stride=k_stride, need_lse=True)
            o, lse = (oi, li) if o is None else merge_partials(o, lse, oi, li)
        if nxt is not None:
            if side is not None:
                main.wait_stream(side)                        # the next chunk has landed before it is read
            kv = nxt
    return o, lse


_RING_STREAMS: dict = {}


def _ring_stream(device):
    key = torch.device(device).index
    if key not in _RING_STREAMS:
        _RING_STREAMS[key] = torch.cuda.Stream(device)
    return _RING_STREAMS[key]


class _FlashBwd(ctypes.Structure):
    _fields_ = [("fwd", _Flash), ("dout", c_void_p), ("delta", c_void_p), ("ld_do", c_longlong), ("do_cols", c_int),
                ("do_col0", c_int), ("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p), ("dk_acc", c_void_p),
                ("dv_acc", c_void_p), ("ld_dq", c_longlong), ("ld_dkv", c_longlong)]


def flash_attention_backward(q, k, v, out, lse, dout, *, causal=True, window=0, scale=None, q_off=0, q_stride=1,
                             k_off=0, k_stride=1, delta=None, dq=None, dkv_acc=None, dropout=None):
    """Gradients of :func:`flash_attention`.  Returns ``(dq fp32 [B,Tq,H,hd], dk, dv)``.

    ``dq`` (fp32) is added to when given.  With ``dkv_acc`` (fp32 ``[2, B, Tk, Hkv, hd]``) the key/value gradients
    are added to it and ``dk, dv`` are returned as its two halves; otherwise they are fresh bf16 tensors.
    ``lse`` must be the log-sum-exp over ALL keys the queries attended to (for ring attention: the merged one),
    and ``delta = rowsum(dout * out)`` of the final output."""
    B, Tq, H, hd = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    scale = hd ** -0.5 if scale is None else scale
    dout = dout.contiguous()
    if delta is None:
        delta = (dout.float() * out.float()).sum(-1).transpose(1, 2).contiguous()       # [B, H, Tq]
    if dq is None:
        dq = torch.zeros((B, Tq, H, hd), dtype=torch.float32, device=q.device)
    if hd not in (64, 128):
        # the backward kernel keeps dK and dV of a key block in tensor memory, which holds them up to 128 columns wide
        return _backward_by_blocks(q, k, v, lse, dout, delta, dq, dkv_acc, causal, window, scale, q_off, q_stride, k_off,
                                   k_stride, dropout)
    a = _FlashBwd()
    f = a.fwd
    f.q, f.ldq, f.q_cols = _view2d(q)
    f.k, f.ldk, f.k_cols = _view2d(k)
    f.v, f.ldv, f.v_cols = _view2d(v)
    f.lse = lse.data_ptr()
    f.B, f.H, f.Hkv, f.Tq, f.Tk, f.head_dim = B, H, Hkv, Tq, Tk, hd
    f.causal, f.window = int(causal), int(window)
    f.q_off, f.q_stride, f.k_off, f.k_stride = q_off, q_stride, k_off, k_stride
    f.scale = scale
    f.status = status_block(q.device).data_ptr()
    _set_dropout(f, dropout)
    a.dout, a.ld_do, a.do_cols = _view2d(dout)
    a.delta = delta.data_ptr()
    a.dq, a.ld_dq = dq.data_ptr(), dq.stride(1)
    if dkv_acc is None:
        dk = torch.empty((B, Tk, Hkv, hd), dtype=torch.bfloat16, device=q.device)
        dv = torch.empty_like(dk)
        a.dk, a.dv, a.ld_dkv = dk.data_ptr(), dv.data_ptr(), dk.stride(1)
    else:
        assert dkv_acc.dtype == torch.float32 and dkv_acc.is_contiguous()
        dk, dv = dkv_acc[0], dkv_acc[1]
        a.dk_acc, a.dv_acc, a.ld_dkv = dk.data_ptr(), dv.data_ptr(), dk.stride(1)
    rc = _native.lib().mesh_flash_attention_bwd(ctypes.byref(a), c_void_p(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "mesh_flash_attention_bwd")
    _native.count_launch()
    return dq, dk, dv


def _backward_by_blocks(q, k, v, lse, dout, delta, dq, dkv_acc, causal, window, scale, q_off, q_stride, k_off, k_stride,
                        dropout, block: int = 512):
    """The attention backward for head sizes the backward kernel does not take (256): the same five products per block
    of queries as the kernel, as fp32 tensor operations (``P = exp(S * scale - L)`` from the forward pass's log-sum-exp,
    ``dS = P (dP - delta) scale``), masks on logical positions.  Memory: one ``[B, H, block, Tk]`` fp32 tile at a time."""
    if dropout is not None and dropout.get("p", 0.0) > 0:
        raise NotImplementedError("attention backward with dropout needs head_dim 64 or 128")
    B, Tq, H, hd = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    kf, vf = k.float(), v.float()
    dk = torch.zeros((B, Tk, Hkv, hd), dtype=torch.float32, device=q.device) if dkv_acc is None else dkv_acc[0]
    dv = torch.zeros_like(dk) if dkv_acc is None else dkv_acc[1]
    kpos = k_off + torch.arange(Tk, device=q.device) * k_stride
    for q0 in range(0, Tq, block):
        q1 = min(Tq, q0 + block)
        qs = q[:, q0:q1].float().view(B, q1 - q0, Hkv, g, hd)
        do = dout[:, q0:q1].float().view(B, q1 - q0, Hkv, g, hd)
        s = torch.einsum("bqhgd,bkhd->bhgqk", qs, kf) * scale
        p = torch.exp(s - lse[:, :, q0:q1].view(B, Hkv, g, q1 - q0, 1).float())
        qpos = q_off + torch.arange(q0, q1, device=q.device) * q_stride
        keep = torch.ones((q1 - q0, Tk), dtype=torch.bool, device=q.device)
        if causal:
            keep &= kpos[None, :] <= qpos[:, None]
        if window and window > 0:
            keep &= kpos[None, :] > qpos[:, None] - window
        p = torch.where(keep, p, torch.zeros((), device=q.device))
        dv += torch.einsum("bhgqk,bqhgd->bkhd", p, do)
        dp = torch.einsum("bqhgd,bkhd->bhgqk", do, vf)
        ds = p * (dp - delta[:, :, q0:q1].view(B, Hkv, g, q1 - q0, 1)) * scale
        dq[:, q0:q1] += torch.einsum("bhgqk,bkhd->bqhgd", ds, kf).reshape(B, q1 - q0, H, hd)
        dk += torch.einsum("bhgqk,bqhgd->bkhd", ds, qs)
    if dkv_acc is None:
        return dq, dk.to(torch.bfloat16), dv.to(torch.bfloat16)
    return dq, dk, dv


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, window, scale, dropout=None):
        out, lse = flash_attention(q, k, v, causal=causal, window=window, scale=scale, need_lse=True, dropout=dropout)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (causal, window, scale, dropout)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        causal, window, scale, dropout = ctx.cfg
        dq, dk, dv = flash_attention_backward(q, k, v, out, lse, dout, causal=causal, window=window, scale=scale,
                                              dropout=dropout)
        return dq.to(q.dtype), dk, dv, None, None, None, None


def attention(q, k, v, *, causal=True, window=0, scale=None, dropout=None):
    """Differentiable attention on the flash kernels (``q [B, T, H, hd]``, ``k, v [B, T, Hkv, hd]``, bf16).
    ``dropout``: ``dict(p=..., seed=..., site=0, execution=0)``; the backward pass redraws the same mask."""
    return _Attention.apply(q, k, v, causal, window, scale, dropout)


def _ring_positions(r, src, P, T, striped):
    return (r, P, src, P) if striped else (r * T, 1, src * T, 1)


class _RingAttention(torch.autograd.Function):
    """Ring attention with its backward: the KV chunks make a second trip around the ring together with fp32
    accumulators of their gradients, each rank adding the part its own queries contribute; one more hop brings
    every accumulator home."""

    @staticmethod
    def forward(ctx, q, k, v, comm, causal, striped, scale, overlap=None):
        out, lse = ring_attention(q, k, v, comm, causal=causal, striped=striped, scale=scale, overlap=overlap)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (comm, causal, striped, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        comm, causal, striped, scale = ctx.cfg
        P, r = comm.world, comm.rank
        B, T, H, hd = q.shape
        dout = dout.contiguous()
        delta = (dout.float() * out.float()).sum(-1).transpose(1, 2).contiguous()
        dq = torch.zeros((B, T, H, hd), dtype=torch.float32, device=q.device)
        kv = torch.stack([k, v]).contiguous()
        dkv = torch.zeros(kv.shape, dtype=torch.float32, device=q.device)
        ring = [(j, (j + 1) % P) for j in range(P)]
        for step in range(P):
            src = (r - step) % P
            q_off, q_stride, k_off, k_stride = _ring_positions(r, src, P, T, striped)
            nxt = None
            if step + 1 < P:
                nxt = torch.empty_like(kv)
                comm.permute(nxt, kv, ring)
            if (not causal) or striped or src <= r:
                flash_attention_backward(q, kv[0], kv[1], out, lse, dout, causal=causal, scale=scale, q_off=q_off,
                                         q_stride=q_stride, k_off=k_off, k_stride=k_stride, delta=delta, dq=dq, dkv_acc=dkv)
            moved = torch.empty_like(dkv)
            comm.permute(moved, dkv, ring)                    # after the last step this hop brings it home
            dkv = moved
            if nxt is not None:
                kv = nxt
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None, None, None


def ring_attention_autograd(q, k, v, comm, *, causal=True, striped=False, scale=None, overlap: bool | None = None):
    """Differentiable :func:`ring_attention` (returns the output only)."""
    return _RingAttention.apply(q, k, v, comm, causal, striped, scale, overlap)


def attention_ref(q, k, v, causal=True, window=0, scale=None, q_off=0, q_stride=1, k_off=0, k_stride=1, dropout=None):
    """fp32 PyTorch statement (oracle)."""
    B, Tq, H, hd = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    scale = hd ** -0.5 if scale is None else scale
    kf = k.float().repeat_interleave(H // Hkv, 2)
    vf = v.float().repeat_interleave(H // Hkv, 2)
    s = torch.einsum("bthd,bshd->bhts", q.float(), kf) * scale
    qp = q_off + torch.arange(Tq, device=q.device) * q_stride
    kp = k_off + torch.arange(Tk, device=q.device) * k_stride
    mask = torch.zeros(Tq, Tk, dtype=torch.bool, device=q.device)
    if causal:
        mask |= kp[None, :] > qp[:, None]
    if window > 0:
        mask |= kp[None, :] <= qp[:, None] - window
    s = s.masked_fill(mask[None, None], float("-inf"))
    lse = torch.logsumexp(s, -1)
    p = torch.softmax(s, -1)
    p = torch.where(torch.isnan(p), torch.zeros_like(p), p)
    if dropout and dropout.get("p"):
        from .philox import attention_keep_mask
        Ht = dropout.get("heads_total") or H
        bh = (torch.arange(B, device=q.device)[:, None] * Ht + dropout.get("head_off", 0) + torch.arange(H, device=q.device)[None, :])
        keep = attention_keep_mask(bh[:, :, None, None], qp[None, None, :, None], kp[None, None, None, :], float(dropout["p"]),
                                   int(dropout.get("seed", 0)), int(dropout.get("site", 0)), int(dropout.get("execution", 0)))
        p = torch.where(keep, p / (1.0 - float(dropout["p"])), torch.zeros_like(p))
    return torch.einsum("bhts,bshd->bthd", p, vf), lse


# ------------------------------------------------------------------------------------------- head-exchange (Ulysses)
def _a2a(x: torch.Tensor, axis) -> torch.Tensor:
    """All-to-all over dim 0 of ``x [P, ...]``: block ``j`` goes to member ``j``; returns ``[P, ...]`` with block ``j``
    received from member ``j``.  ``axis``: an axis context (own kernels on CUDA with a heap) or a torch group."""
    import torch.distributed as dist
    x = x.contiguous()
    out = torch.empty_like(x)
    comm = getattr(axis, "comm", None) if (x.is_cuda and getattr(axis, "_heap", None) is not None) else None
    if comm is not None:
        comm.all_to_all(out.view(x.shape[0], -1), x.view(x.shape[0], -1))
    else:
        dist.all_to_all_single(out, x, group=getattr(axis, "group", axis))
    return out


class _SeqToHeads(torch.autograd.Function):
    """``[B, T/P, H, hd]`` (sequence cut) -> ``[B, T, H/P, hd]`` (heads cut); the backward is the inverse exchange."""

    @staticmethod
    def forward(ctx, x, axis, P):
        ctx.axis, ctx.P = axis, P
        B, Tl, H, hd = x.shape
        send = x.view(B, Tl, P, H // P, hd).permute(2, 0, 1, 3, 4)            # [P(dst), B, Tl, H/P, hd]
        got = _a2a(send, axis)                                                  # [P(src = sequence block), B, Tl, H/P, hd]
        return got.permute(1, 0, 2, 3, 4).reshape(B, P * Tl, H // P, hd)

    @staticmethod
    def backward(ctx, g):
        return _HeadsToSeq.apply(g, ctx.axis, ctx.P), None, None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, axis, P):
        ctx.axis, ctx.P = axis, P
        B, T, Hl, hd = x.shape
        send = x.view(B, P, T // P, Hl, hd).permute(1, 0, 2, 3, 4)             # [P(dst = owner of the block), B, Tl, Hl, hd]
        got = _a2a(send, axis)                                                  # [P(src = head group), B, Tl, Hl, hd]
        return got.permute(1, 2, 0, 3, 4).reshape(B, T // P, P * Hl, hd)

    @staticmethod
    def backward(ctx, g):
        return _SeqToHeads.apply(g, ctx.axis, ctx.P), None, None


def ulysses_attention(q, k, v, axis, *, causal=True, window=0, scale=None, local_attention=None):
    """Context-parallel attention by exchanging heads for sequence: every member holds a contiguous ``T / P`` slice
    of the tokens for all heads; one all-to-all gives it all tokens of ``H / P`` heads, attention runs locally on whole
    sequences, and a second all-to-all restores the sequence cut.  Needs ``H`` (and the KV heads) divisible by ``P``;
    costs two all-to-alls of the activations instead of ``P - 1`` KV rotations, which wins when there are enough heads.
    The reference reaches this form through its generic all-to-all reshard (compiler/mesh_compiler/placement.py:270).
    Differentiable.  ``local_attention(q, k, v)`` defaults to the flash kernels on CUDA bf16 and to the fp32
    statement elsewhere."""
    P = axis.world
    if P == 1:
        qh, kh, vh = q, k, v
    else:
        if q.shape[2] % P or k.shape[2] % P:
            raise ValueError("head-exchange attention needs the query and KV heads divisible by the group size")
        qh, kh, vh = (_SeqToHeads.apply(t, axis, P) for t in (q, k, v))
    if local_attention is None:
        if qh.is_cuda and qh.dtype == torch.bfloat16:
            local_attention = lambda a, b, c: attention(a, b, c, causal=causal, window=window, scale=scale)
        else:
            local_attention = lambda a, b, c: attention_ref(a, b, c, causal, window, scale)[0].to(a.dtype)
    oh = local_attention(qh, kh, vh)
    return oh if P == 1 else _HeadsToSeq.apply(oh, axis, P)
