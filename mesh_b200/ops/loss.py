"""Scalar reductions a training loop reads every step, as one kernel each."""
from __future__ import annotations

from ctypes import c_longlong, c_void_p

import torch

from .. import _native

_scratch: dict = {}


def dot_sum(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``sum(a * b)`` of two bf16 CUDA tensors of equal shape as a 0-d fp32 tensor (fp32 accumulation).

    With fixed ``b`` this is the loss whose gradient with respect to ``a`` is ``b``: a step that seeds its backward
    pass with ``b`` can report the loss with this one launch.  The tensor-op formulation
    ``(a.float() * b.float()).sum()`` takes four launches and two fp32 temporaries."""
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or not a.is_cuda or a.shape != b.shape:
        raise ValueError("dot_sum: expected two bf16 CUDA tensors of the same shape")
    a, b = a.contiguous(), b.contiguous()
    L = _native.lib()
    key = (a.device.index, torch.cuda.current_stream(a.device).cuda_stream)
    if key not in _scratch:
        _scratch[key] = (torch.empty(L.mesh_dot_sum_blocks(), dtype=torch.float32, device=a.device),
                         torch.zeros(1, dtype=torch.int32, device=a.device))
    partials, ticket = _scratch[key]
    if out is None:
        out = torch.empty((), dtype=torch.float32, device=a.device)
    rc = L.mesh_dot_sum_bf16(c_void_p(a.data_ptr()), c_void_p(b.data_ptr()), c_longlong(a.numel()),
                             c_void_p(out.data_ptr()), c_void_p(partials.data_ptr()), c_void_p(ticket.data_ptr()),
                             c_void_p(torch.cuda.current_stream(a.device).cuda_stream))
    _native.check(rc, "mesh_dot_sum_bf16")
    _native.count_launch()
    return out
