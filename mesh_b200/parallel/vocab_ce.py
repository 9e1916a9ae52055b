"""Cross-entropy over logits whose vocabulary dimension is cut over a tensor-parallel axis.

With the output projection column-parallel every rank holds ``logits[:, v0:v1]`` for its slice of the vocabulary.  The
loss needs three per-token statistics of the whole row - the maximum, the sum of exponentials and the target's logit -
so two tiny all-reduces (a max of ``N`` floats, then a sum of ``2N`` floats) replace the all-gather of ``N x V`` logits
(the reference states the pieces as online max / sum statistics, compiler/mesh_compiler/operations.py:6281-6330, and
its vocabulary-parallel embedding as a masked lookup followed by a sum, placement.py:812-834).  The backward needs no
communication: ``d logits = (softmax - onehot) * d loss`` on the local columns.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .collectives_autograd import _comm_of, _world


def _all_reduce(x: torch.Tensor, group, op: str) -> None:
    if _world(group) == 1:
        return
    comm, g = _comm_of(group, x)
    if comm is not None:
        comm.all_reduce(x, op=op)
    else:
        dist.all_reduce(x, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM, group=g)


def _s():
    from ctypes import c_void_p
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class _VocabParallelCEKernel(torch.autograd.Function):
    """bf16 CUDA logits: statistics in one pass (``csrc/ops/cross_entropy.cu``), two tiny all-reduces, gradient in one
    pass from the logits themselves - no fp32 copy of the logits or of their exponentials is kept for the backward."""

    @staticmethod
    def forward(ctx, logits, targets, start, group, ignore_index):
        from ctypes import c_int, c_longlong, c_void_p
        from .. import _native
        n, v = logits.shape
        dev = logits.device
        t64 = targets.to(torch.int64).contiguous()
        stats = torch.empty((3, n), dtype=torch.float32, device=dev)            # local max, local sum, target logit
        rc = _native.lib().mesh_ce_stats_bf16(c_void_p(logits.data_ptr()), c_longlong(logits.stride(0)), c_int(n), c_int(v),
                                              c_void_p(t64.data_ptr()), c_longlong(start), c_longlong(ignore_index),
                                              c_void_p(stats[0].data_ptr()), c_void_p(stats[1].data_ptr()),
                                              c_void_p(stats[2].data_ptr()), _s())
        _native.check(rc, "mesh_ce_stats_bf16")
        _native.count_launch()
        gmax = stats[0].clone()
        _all_reduce(gmax, group, "max")
        sums = torch.stack([stats[1] * torch.exp(stats[0] - gmax), stats[2]])
        _all_reduce(sums, group, "sum")
        live = t64 != ignore_index
        loss = torch.where(live, torch.log(sums[0]) + gmax - sums[1], torch.zeros_like(gmax))
        ctx.save_for_backward(logits, t64, gmax, sums[0].contiguous(), live)
        ctx.start = start
        return loss

    @staticmethod
    def backward(ctx, g):
        from ctypes import c_int, c_longlong, c_void_p
        from .. import _native
        logits, t64, gmax, gsum, live = ctx.saved_tensors
        n, v = logits.shape
        gscale = (g.float() * live.float()).contiguous()
        d = torch.empty((n, v), dtype=torch.bfloat16, device=logits.device)
        rc = _native.lib().mesh_ce_grad_bf16(c_void_p(logits.data_ptr()), c_longlong(logits.stride(0)), c_void_p(d.data_ptr()),
                                             c_longlong(d.stride(0)), c_int(n), c_int(v), c_void_p(t64.data_ptr()),
                                             c_longlong(ctx.start), c_void_p(gmax.data_ptr()), c_void_p(gsum.data_ptr()),
                                             c_void_p(gscale.data_ptr()), _s())
        _native.check(rc, "mesh_ce_grad_bf16")
        _native.count_launch()
        return d, None, None, None, None


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, start, group, ignore_index):
        x = logits.float()
        n, v = x.shape
        row_max = x.max(-1).values
        _all_reduce(row_max, group, "max")
        ex = torch.exp(x - row_max[:, None])
        local = targets - start
        mine = (local >= 0) & (local < v) & (targets != ignore_index)
        at = local.clamp(0, v - 1)
        stats = torch.stack([ex.sum(-1), torch.where(mine, x.gather(1, at[:, None])[:, 0], torch.zeros_like(row_max))])
        _all_reduce(stats, group, "sum")
        sum_exp, target_logit = stats[0], stats[1]
        live = targets != ignore_index
        loss = torch.where(live, torch.log(sum_exp) + row_max - target_logit, torch.zeros_like(row_max))
        ctx.save_for_backward(ex, sum_exp, at, mine, live)
        ctx.dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        ex, sum_exp, at, mine, live = ctx.saved_tensors
        grad = ex / sum_exp[:, None]
        grad.scatter_add_(1, at[:, None], -mine.to(grad.dtype)[:, None])
        grad = grad * (g * live.to(g.dtype))[:, None]
        return grad.to(ctx.dtype), None, None, None, None


def vocab_parallel_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int, group=None,
                                 ignore_index: int = -100, reduction: str = "mean") -> torch.Tensor:
    """``logits [N, V_local]``: this rank's columns ``vocab_start : vocab_start + V_local`` of every token's logits;
    ``targets [N]``: global class ids (the same on every rank of ``group``, a torch.distributed group or an axis
    context).  Returns the per-token losses (``reduction="none"``), their sum, or their mean over the tokens that are
    not ``ignore_index``."""
    if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.dim() == 2 and logits.stride(1) == 1:
        loss = _VocabParallelCEKernel.apply(logits, targets, int(vocab_start), group, int(ignore_index))
    else:
        loss = _VocabParallelCE.apply(logits, targets, int(vocab_start), group, int(ignore_index))
    if reduction == "none":
        return loss
    if reduction == "sum":
        return loss.sum()
    return loss.sum() / (targets != ignore_index).sum().clamp(min=1)


class VocabParallelHead(torch.nn.Module):
    """Output projection with the vocabulary cut over ``group`` and the loss computed without gathering the logits."""

    def __init__(self, d_model: int, vocab: int, rank: int, world: int, group=None, dtype=torch.float32, device=None,
                 init_std: float = 0.02, seed: int = 7):
        super().__init__()
        if vocab % world:
            raise ValueError("the vocabulary must divide over the axis")
        self.group, self.start, self.rows = group, rank * (vocab // world), vocab // world
        g = torch.Generator(device="cpu").manual_seed(seed)
        full = torch.empty(vocab, d_model).normal_(0, init_std, generator=g)
        self.weight = torch.nn.Parameter(full[self.start:self.start + self.rows].to(device=device, dtype=dtype))

    def forward(self, h: torch.Tensor, targets: torch.Tensor, reduction: str = "mean") -> torch.Tensor:
        """``h [N, d_model]`` (the same on every rank of the axis; its gradient is summed over the axis)."""
        from .collectives_autograd import copy_to_tp
        if _world(self.group) > 1:
            h = copy_to_tp(h, self.group)
        logits = torch.nn.functional.linear(h, self.weight)
        return vocab_parallel_cross_entropy(logits, targets, self.start, self.group, reduction=reduction)
