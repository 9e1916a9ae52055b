"""Tensor-parallel layers (public API).

The reference has no layer classes — its "layer library" is placement functions over an exported
graph (``megatron()``, examples/parallel.py:77-89).  These modules are the eager counterpart with the
same sharding: column-parallel gate/up, row-parallel down, sequence-sharded activations.  On CUDA
they run the fused compute+collective kernels; on CPU (gloo ranks) the same math runs through
torch ops and the process group, which is what the plumbing tests use.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..distributed.context import MeshContext, context


def _act(name: str):
    return F.silu if name in ("silu", "swiglu") else (lambda t: F.gelu(t, approximate="tanh"))


class TPGatedFFN(nn.Module):
    """SwiGLU / GeGLU FFN split over ``ctx.world`` ranks.

    ``sequence_parallel=True``: input and output are this rank's ``[tokens/world, d_model]`` shard
    (all-gather before, reduce-scatter after).  ``False``: input replicated, output all-reduced.
    Parameters hold only this rank's shard: ``w_gate_up [2*d_ff/world, d_model]`` (gate rows then up
    rows) and ``w_down [d_model, d_ff/world]``.  ``ff_shares``: hidden units per rank when the ranks are not alike (any
    multiples of 64 that add up to ``d_ff``; e.g. from ``runtime/allocate.py``), instead of equal shares.
    """

    def __init__(self, d_model: int, d_ff: int, ctx: MeshContext | None = None, act: str = "silu",
                 sequence_parallel: bool = True, dtype=torch.bfloat16, device=None, init_std: float = 0.02,
                 seed: int = 0, in_flight: int = 1, ff_shares=None):
        super().__init__()
        self.ctx = ctx or context()
        P, r = self.ctx.world, self.ctx.rank
        if ff_shares is None:
            assert d_ff % P == 0
            ff_shares = [d_ff // P] * P
        ff_shares = [int(v) for v in ff_shares]
        if len(ff_shares) != P or sum(ff_shares) != d_ff or any(v <= 0 for v in ff_shares):
            raise ValueError(f"ff_shares {ff_shares} must give every one of {P} ranks a positive share adding up to {d_ff}")
        self.ff_shares = ff_shares
        self.d_model, self.d_ff, self.act, self.sp = d_model, d_ff, act, sequence_parallel
        device = device or self.ctx.device
        # Every rank draws the full matrices from the same seed and keeps its slice, so a TP=P model
        # equals the TP=1 model with the same seed (the reference seeds every rank alike,
        # examples/parallel.py:223-226, but keeps whole copies; here only the shard is materialised
        # on the device).
        g = torch.Generator(device="cpu").manual_seed(seed)
        lo, hi = sum(ff_shares[:r]), sum(ff_shares[:r + 1])
        wg = torch.empty(d_ff, d_model).normal_(0, init_std, generator=g)[lo:hi]
        wu = torch.empty(d_ff, d_model).normal_(0, init_std, generator=g)[lo:hi]
        wd = torch.empty(d_model, d_ff).normal_(0, init_std, generator=g)[:, lo:hi]
        self.w_gate_up = nn.Parameter(torch.cat([wg, wu], 0).to(device=device, dtype=dtype))
        self.w_down = nn.Parameter(wd.contiguous().to(device=device, dtype=dtype))
        self._fused = None
        self._fused_tokens = None
        self.in_flight = in_flight          # forward passes that may run before their backward passes (pipeline microbatches)

    def _fused_op(self, tokens_total: int):
        if self._fused is None or self._fused_tokens != tokens_total:
            from .tp_ffn import FusedTPFFN
            self._fused = FusedTPFFN(self.ctx.heap, tokens_total, self.d_model, self.d_ff, self.act, in_flight=self.in_flight,
                                     ff_local=self.ff_shares[self.ctx.rank])
            self._fused_tokens = tokens_total
        return self._fused

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        P = self.ctx.world
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.d_model)
        if x2.is_cuda and x2.dtype == torch.bfloat16:
            if P == 1:
                from ..ops.gemm import glu_ffn
                return glu_ffn(x2, self.w_gate_up, self.w_down, self.act).reshape(*lead, self.d_model)
            if self.sp:
                from .tp_ffn import fused_tp_ffn
                op = self._fused_op(x2.shape[0] * P)
                return fused_tp_ffn(x2.contiguous(), self.w_gate_up, self.w_down, op).reshape(*lead, self.d_model)
        # torch-op path (CPU ranks, fp32, or replicated activations)
        from .collectives_autograd import all_gather_seq, all_reduce_sum, copy_to_tp, reduce_scatter_seq
        Fl = self.ff_shares[self.ctx.rank]
        if P > 1:
            x2 = all_gather_seq(x2, self.ctx.group) if self.sp else copy_to_tp(x2, self.ctx.group)
        gate = F.linear(x2, self.w_gate_up[:Fl])
        up = F.linear(x2, self.w_gate_up[Fl:])
        y = F.linear(_act(self.act)(gate) * up, self.w_down)
        if P > 1:
            y = reduce_scatter_seq(y, self.ctx.group) if self.sp else all_reduce_sum(y, self.ctx.group)
        return y.reshape(*lead[:-1], -1, self.d_model) if len(lead) > 1 and not self.sp else y
