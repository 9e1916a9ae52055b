"""Sharded AdamW: bf16 parameters, fp32 master weights and moments held only for this rank's shard.

Tensor-parallel parameters are already shards; with ``dp_group`` the state of replicated parameters is cut over
the data-parallel ranks too (ZeRO-1): gradients are reduce-scattered, each rank updates its slice with the fused
kernel (csrc/ops/adamw.cu) and the updated bf16 slices are all-gathered.  On CPU the same arithmetic runs in torch.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch
import torch.distributed as dist


class ShardedAdamW:
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, dp_group=None, dp_world: int = 1,
                 dp_rank: int = 0):
        self.params = [p for p in params]
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.group, self.W, self.r = dp_group, dp_world, dp_rank
        self.step_no = 0
        self.state = []
        for p in self.params:
            n = p.numel()
            per = -(-n // self.W)
            lo, hi = min(n, self.r * per), min(n, (self.r + 1) * per)
            master = p.detach().reshape(-1)[lo:hi].float().clone()
            self.state.append({"lo": lo, "hi": hi, "per": per, "master": master, "m": torch.zeros_like(master),
                               "v": torch.zeros_like(master)})

    def _update(self, st, g, out_bf16):
        self_step = self.step_no
        b1, b2 = self.betas
        if st["master"].is_cuda:
            from .. import _native
            rc = _native.lib().mesh_adamw_step(c_void_p(st["master"].data_ptr()), c_void_p(st["m"].data_ptr()),
                                               c_void_p(st["v"].data_ptr()), c_void_p(g.data_ptr()),
                                               c_int(int(g.dtype == torch.bfloat16)),
                                               c_void_p(out_bf16.data_ptr() if out_bf16 is not None else 0),
                                               c_longlong(st["master"].numel()), c_float(self.lr), c_float(b1), c_float(b2),
                                               c_float(self.eps), c_float(self.wd), c_int(self_step), c_float(1.0),
                                               c_void_p(torch.cuda.current_stream().cuda_stream))
            _native.check(rc, "mesh_adamw_step")
            _native.count_launch()
            return
        g = g.float()
        st["m"].mul_(b1).add_(g, alpha=1 - b1)
        st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
        mhat = st["m"] / (1 - b1 ** self_step)
        vhat = st["v"] / (1 - b2 ** self_step)
        st["master"].mul_(1 - self.lr * self.wd).addcdiv_(mhat, vhat.sqrt() + self.eps, value=-self.lr)
        if out_bf16 is not None:
            out_bf16.copy_(st["master"])

    @torch.no_grad()
    def step(self, grads: list | None = None):
        """``grads[i]`` (default ``p.grad``): the full gradient when ``dp_world == 1`` or already-summed gradients;
        with a data-parallel group the local gradients are reduce-scattered here."""
        self.step_no += 1
        for i, (p, st) in enumerate(zip(self.params, self.state)):
            g = (grads[i] if grads is not None else p.grad).reshape(-1)
            n, per = p.numel(), st["per"]
            if self.W > 1:
                pad = per * self.W - n
                gp = torch.cat([g, g.new_zeros(pad)]) if pad else g
                mine = torch.empty(per, dtype=g.dtype, device=g.device)
                dist.reduce_scatter_tensor(mine, gp.contiguous(), group=self.group)
                mine = mine[: st["hi"] - st["lo"]] / self.W
                new = torch.empty(per, dtype=p.dtype, device=p.device)
                self._update(st, mine.contiguous(), None)
                new[: st["hi"] - st["lo"]] = st["master"].to(p.dtype)
                full = torch.empty(per * self.W, dtype=p.dtype, device=p.device)
                dist.all_gather_into_tensor(full, new, group=self.group)
                p.copy_(full[:n].view_as(p))
            else:
                flat = p.view(-1) if p.is_contiguous() else None
                if p.dtype == torch.bfloat16 and flat is not None and p.is_cuda:
                    self._update(st, g.contiguous(), flat)
                else:
                    self._update(st, g.contiguous(), None)
                    p.copy_(st["master"].view_as(p).to(p.dtype))

    def state_dict(self) -> dict:
        out = {"step": self.step_no}
        for i, st in enumerate(self.state):
            out[f"master.{i}"], out[f"m.{i}"], out[f"v.{i}"] = st["master"], st["m"], st["v"]
        return out

    def load_state_dict(self, sd: dict) -> None:
        self.step_no = int(sd["step"])
        for i, st in enumerate(self.state):
            st["master"].copy_(sd[f"master.{i}"]); st["m"].copy_(sd[f"m.{i}"]); st["v"].copy_(sd[f"v.{i}"])


class BucketedAdamW:
    """ZeRO-1 AdamW over the buckets of a :class:`~mesh_b200.parallel.dp.DataParallel`.

    The gradient traffic is the data-parallel wrapper's: one reduce-scatter per bucket, started from the autograd hooks
    while the backward pass is still running, on this package's collective kernels when the ranks share a symmetric
    heap.  This optimizer holds fp32 master weights and moments for this rank's slice of every bucket only, updates
    the slice with the fused kernel (which also writes the new bf16 values) and all-gathers the updated slices, one
    all-gather per bucket - no per-parameter collectives.  ``dp`` must be built with ``all_reduce=False``."""

    def __init__(self, dp, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0):
        if dp.all_reduce:
            raise ValueError("BucketedAdamW reduces and gathers the buckets itself: build DataParallel(all_reduce=False)")
        self.dp = dp
        self._inner = ShardedAdamW([], lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self.state = []
        for b in dp.buckets:
            flat = torch.cat([p.detach().reshape(-1) for p in b.params])
            if b.padded > flat.numel():
                flat = torch.cat([flat, flat.new_zeros(b.padded - flat.numel())])
            lo = dp.rank * b.per
            master = flat[lo:lo + b.per].float().clone()
            self.state.append({"master": master, "m": torch.zeros_like(master), "v": torch.zeros_like(master),
                               "new": torch.empty(b.per, dtype=b.params[0].dtype, device=master.device)})

    @property
    def step_no(self) -> int:
        return self._inner.step_no

    @torch.no_grad()
    def step(self) -> None:
        """After ``loss.backward()``: joins the bucket reductions, updates, gathers."""
        shards = self.dp.finish()
        self._inner.step_no += 1
        for b, st, (_, g) in zip(self.dp.buckets, self.state, shards):
            new = st["new"]
            if st["master"].is_cuda and new.dtype == torch.bfloat16:
                self._inner._update(st, g.contiguous(), new)
            else:
                self._inner._update(st, g.contiguous(), None)
                new.copy_(st["master"])
            full = self.dp.all_gather(new) if self.dp.world > 1 else new
            for p, off in zip(b.params, b.offsets):
                p.copy_(full[off: off + p.numel()].view_as(p))

    def state_dict(self) -> dict:
        out = {"step": self._inner.step_no}
        for i, st in enumerate(self.state):
            out[f"master.{i}"], out[f"m.{i}"], out[f"v.{i}"] = st["master"], st["m"], st["v"]
        return out

    def load_state_dict(self, sd: dict) -> None:
        self._inner.step_no = int(sd["step"])
        for i, st in enumerate(self.state):
            st["master"].copy_(sd[f"master.{i}"]); st["m"].copy_(sd[f"m.{i}"]); st["v"].copy_(sd[f"v.{i}"])
