"""Attention as one differentiable operator of training graphs: ``mesh::attention`` and ``mesh::attention_backward``.

A joint forward+backward capture has to expand ``scaled_dot_product_attention`` (it is a composite without a backward
node of its own), and the plain expansion leaves a dozen products, masks and softmax pieces per attention, forward and
backward, for the placement to carry a cut through and for the executor to run one by one.  The reference keeps
attention one operator with a forward and a backward (blockwise, with the row statistics kept from the forward;
compiler/mesh_compiler/operations.py:7081-7166); so do these two:

    out, lse = mesh::attention(q, k, v, causal, scale, row_start, row_step)
    dq, dk, dv = mesh::attention_backward(grad, q, k, v, out, lse, causal, scale, row_start, row_step)

``q`` is ``[batch, heads, queries, head_dim]``, ``k`` / ``v`` ``[batch, kv_heads, keys, head_dim]`` (``heads`` a multiple
of ``kv_heads``); ``lse`` is the log of every row's sum of exponentials (fp32), from which the backward recomputes the
probabilities instead of keeping them.  With ``causal``, query ``i`` sits at position ``row_start + i * row_step`` of the
whole sequence and sees the keys up to that position: a processor that holds a block (``row_step`` 1) or every
``row_step``-th query (a round-robin share) of the queries states where they are, which is how the placement keeps the
queries cut along the sequence.  The capture stage substitutes the operator for attention calls without a mask tensor
and without dropout (``compiler/export.py``); the arithmetic is fp32 inside, in PyTorch operators on any device.
"""
from __future__ import annotations

import torch

_lib = torch.library.Library("mesh", "FRAGMENT")
_lib.define("attention(Tensor q, Tensor k, Tensor v, bool causal, float scale, int row_start, int row_step) -> (Tensor, Tensor)")
_lib.define("attention_backward(Tensor grad, Tensor q, Tensor k, Tensor v, Tensor out, Tensor lse, bool causal, float scale, "
            "int row_start, int row_step) -> (Tensor, Tensor, Tensor)")


def _scores(q, k, causal, scale, row_start, row_step):
    group = q.shape[1] // k.shape[1] if k.shape[1] else 1
    kk = k.float()
    if group > 1:
        kk = kk.repeat_interleave(group, 1)
    s = (q.float() @ kk.transpose(-1, -2)) * scale
    if causal:
        qpos = row_start + row_step * torch.arange(q.shape[2], device=q.device)
        kpos = torch.arange(k.shape[2], device=q.device)
        s = s.masked_fill(kpos[None, :] > qpos[:, None], float("-inf"))
    return s, kk, group


def _probabilities(s, lse):
    finite = torch.isfinite(lse)[..., None]
    return torch.where(finite, torch.exp(s - torch.where(finite, lse[..., None], torch.zeros_like(lse[..., None]))),
                       torch.zeros_like(s))                 # a row that sees no key has no weights


def _forward(q, k, v, causal, scale, row_start, row_step):
    s, _kk, group = _scores(q, k, causal, scale, row_start, row_step)
    lse = torch.logsumexp(s, -1)
    p = _probabilities(s, lse)
    vv = v.float()
    if group > 1:
        vv = vv.repeat_interleave(group, 1)
    return (p @ vv).to(q.dtype), lse


def _backward(grad, q, k, v, out, lse, causal, scale, row_start, row_step):
    s, kk, group = _scores(q, k, causal, scale, row_start, row_step)
    p = _probabilities(s, lse)
    g = grad.float()
    vv = v.float()
    if group > 1:
        vv = vv.repeat_interleave(group, 1)
    dv = p.transpose(-1, -2) @ g
    dp = g @ vv.transpose(-1, -2)
    delta = (g * out.float()).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ kk
    dk = ds.transpose(-1, -2) @ q.float()
    if group > 1:                                           # the heads of a group share their keys and values
        B, H, T, D = dk.shape
        dk = dk.view(B, H // group, group, T, D).sum(2)
        dv = dv.view(B, H // group, group, T, dv.shape[-1]).sum(2)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


_lib.impl("attention", _forward, "CompositeExplicitAutograd")
_lib.impl("attention_backward", _backward, "CompositeExplicitAutograd")


@torch.library.register_fake("mesh::attention")
def _attention_fake(q, k, v, causal, scale, row_start, row_step):
    return q.new_empty((*q.shape[:-1], v.shape[-1])), q.new_empty(q.shape[:-1], dtype=torch.float32)


@torch.library.register_fake("mesh::attention_backward")
def _attention_backward_fake(grad, q, k, v, out, lse, causal, scale, row_start, row_step):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _setup(ctx, inputs, output):
    q, k, v, causal, scale, row_start, row_step = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse)
    ctx.rest = (causal, scale, row_start, row_step)


def _differentiate(ctx, grad_out, _grad_lse):
    q, k, v, out, lse = ctx.saved_tensors
    dq, dk, dv = torch.ops.mesh.attention_backward(grad_out, q, k, v, out, lse, *ctx.rest)
    return dq, dk, dv, None, None, None, None


torch.library.register_autograd("mesh::attention", _differentiate, setup_context=_setup)

FORWARD = torch.ops.mesh.attention.default
BACKWARD = torch.ops.mesh.attention_backward.default


def substitute(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None, enable_gqa=False):
    """What ``scaled_dot_product_attention`` becomes in a training capture: the operator above when there is neither a
    mask tensor nor dropout (and the heads group evenly), the plain formulation in products and a softmax otherwise."""
    plain = attn_mask is None and not dropout_p and query.dim() == 4 and key.dim() == 4 and \
        key.shape[1] > 0 and query.shape[1] % key.shape[1] == 0 and (enable_gqa or query.shape[1] == key.shape[1])
    if plain:
        sc = float(query.shape[-1] ** -0.5) if scale is None else float(scale)
        return torch.ops.mesh.attention(query, key, value, bool(is_causal), sc, 0, 1)[0]
    if attn_mask is not None and attn_mask.dtype == torch.bool:        # the plain formulation takes an additive mask
        attn_mask = torch.zeros_like(attn_mask, dtype=query.dtype).masked_fill(attn_mask.logical_not(), float("-inf"))
    return torch.ops.aten._scaled_dot_product_attention_math.default(query, key, value, attn_mask, dropout_p, is_causal,
                                                                      scale=scale, enable_gqa=enable_gqa)[0]
