"""MoE router: softmax over experts + top-k, one warp per token.

Reference: ``softmax(x @ W_r).topk(k)`` in examples/ep.py:15-22.
"""
from __future__ import annotations

from ctypes import c_int, c_void_p

import torch

from .. import _native


def router_topk(logits: torch.Tensor, k: int, bias: torch.Tensor | None = None, renorm: bool = True):
    """Returns ``(weights fp32 [T,k], indices int32 [T,k])``; ties go to the lower expert index."""
    assert logits.is_cuda and logits.dim() == 2 and logits.is_contiguous()
    assert logits.dtype in (torch.float32, torch.bfloat16)
    T, E = logits.shape
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    rc = _native.lib().mesh_router_topk(c_void_p(logits.data_ptr()), c_int(int(logits.dtype == torch.float32)),
                                        c_void_p(0 if bias is None else bias.data_ptr()), c_void_p(w.data_ptr()),
                                        c_void_p(idx.data_ptr()), c_int(T), c_int(E), c_int(k), c_int(int(renorm)),
                                        c_void_p(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "mesh_router_topk")
    _native.count_launch(1)
    return w, idx


def router_topk_ref(logits: torch.Tensor, k: int, bias: torch.Tensor | None = None, renorm: bool = True):
    x = logits.float()
    if bias is not None:
        x = x + bias.float()
    p = torch.softmax(x, dim=-1)
    w, i = torch.topk(p, k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return w, i.to(torch.int32)
