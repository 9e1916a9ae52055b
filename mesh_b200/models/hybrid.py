"""A decoder-only transformer trained under tensor x context x pipeline x data parallelism at once.

Sharding per axis (the reference states the same cuts as placements over an exported graph: ``megatron()`` splits
the head and hidden dimensions, examples/parallel.py:77-89; striped tokens for causal attention,
compiler/mesh_compiler/placement.py:57-69; layers on different processors, examples/engines.py:91-96):

* **tp** - attention heads and the FFN hidden dimension; activations between sub-layers are sharded over the
  tokens too (sequence parallel), so a sub-layer is all-gather -> column-parallel GEMM ... row-parallel GEMM ->
  reduce-scatter.  The FFN runs the fused compute+collective kernels; the attention projections use the
  axis' collectives around the plain GEMM.
* **cp** - the sequence: each rank owns ``T / cp`` tokens of every sample (striped ``r, r + cp, ...`` by default, so
  causal work is balanced) and attention runs as a ring over the axis.
* **pp** - contiguous runs of layers; one-forward-one-backward over microbatches (``parallel/pp.py``).
* **dp** - the batch; gradients are averaged over the axis and the optimiser state is cut over it.

On CPU ranks the same program runs in fp32 through torch ops and gloo, which is how the sharding logic is tested
against the single-process model.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..parallel.collectives_autograd import all_gather_seq, all_reduce_sum, reduce_scatter_seq
from ..parallel.layers import TPGatedFFN
from ..parallel.pp import run_1f1b, split_layers
from ..parallel.topology import ParallelContext, ParallelDims


@dataclass
class HybridConfig:
    vocab: int = 4096
    d_model: int = 1024
    n_layers: int = 4
    n_heads: int = 8
    n_kv_heads: int = 4
    head_dim: int = 128
    d_ff: int = 4096
    seq_len: int = 1024
    rope_theta: float = 10000.0
    eps: float = 1e-6
    striped: bool = True
    act: str = "silu"
    init_std: float = 0.02


def _fast(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def _norm(x, w, eps):
    if _fast(x):
        from ..ops.norm import rmsnorm
        return rmsnorm(x, w, eps)
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def _linear(x, w):
    if _fast(x):
        from ..ops.gemm import linear
        return linear(x, w)
    return F.linear(x, w)


def _rope_torch(x, pos, theta):
    """x [B, T, H, hd]; rotate-half convention."""
    hd = x.shape[-1]
    inv = theta ** (-torch.arange(0, hd, 2, device=x.device, dtype=torch.float32) / hd)
    ang = pos.float()[:, None] * inv[None]
    cos, sin = ang.cos()[None, :, None], ang.sin()[None, :, None]
    x1, x2 = x[..., : hd // 2].float(), x[..., hd // 2:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


class _GatherKV(torch.autograd.Function):
    """All-gather along the token dimension of ``[B, T, H, hd]`` with a reduce-scatter backward (CPU ring stand-in)."""

    @staticmethod
    def forward(ctx, x, group, world):
        ctx.group, ctx.world = group, world
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.stack(parts, 0)                         # [cp, B, T, H, hd]

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g[dist.get_rank(ctx.group)].clone(), None, None


class Attention(nn.Module):
    def __init__(self, cfg: HybridConfig, par: ParallelContext, layer: int, dtype, device, in_flight: int = 1):
        super().__init__()
        self.cfg, self.par, self.in_flight = cfg, par, in_flight
        self._fused = {}
        tp = par.tp
        assert cfg.n_heads % tp.world == 0 and cfg.n_kv_heads % tp.world == 0, "heads must divide over tp"
        self.Hq, self.Hkv, self.hd = cfg.n_heads // tp.world, cfg.n_kv_heads // tp.world, cfg.head_dim
        g = torch.Generator(device="cpu").manual_seed(1000 + layer)
        D, hd = cfg.d_model, cfg.head_dim
        wq = torch.empty(cfg.n_heads * hd, D).normal_(0, cfg.init_std, generator=g)
        wk = torch.empty(cfg.n_kv_heads * hd, D).normal_(0, cfg.init_std, generator=g)
        wv = torch.empty(cfg.n_kv_heads * hd, D).normal_(0, cfg.init_std, generator=g)
        wo = torch.empty(D, cfg.n_heads * hd).normal_(0, cfg.init_std / math.sqrt(2 * cfg.n_layers), generator=g)
        r = tp.rank
        qs, ks = slice(r * self.Hq * hd, (r + 1) * self.Hq * hd), slice(r * self.Hkv * hd, (r + 1) * self.Hkv * hd)
        self.w_qkv = nn.Parameter(torch.cat([wq[qs], wk[ks], wv[ks]], 0).to(device=device, dtype=dtype))
        self.w_o = nn.Parameter(wo[:, qs].contiguous().to(device=device, dtype=dtype))
        self._rope = None

    def _tables(self, device):
        if self._rope is None:
            from ..ops.rope import rope_tables
            self._rope = rope_tables(self.cfg.seq_len, self.hd, self.cfg.rope_theta, device=device)
        return self._rope

    def _fused_ops(self, tokens: int):
        """The fused projection kernels for ``tokens`` rows over the tensor axis (None when the shape does not fit)."""
        if tokens not in self._fused:
            tp = self.par.tp
            nq = (self.Hq + 2 * self.Hkv) * self.hd
            ok = tokens % (tp.world * 128) == 0 and nq % 64 == 0 and (self.Hq * self.hd) % 64 == 0 and self.cfg.d_model % 64 == 0
            if ok:
                from ..parallel.fused_linear import FusedColumnLinear, FusedRowLinear
                self._fused[tokens] = (FusedColumnLinear(tp.heap, tokens, self.cfg.d_model, nq, in_flight=self.in_flight),
                                       FusedRowLinear(tp.heap, tokens, self.Hq * self.hd, self.cfg.d_model))
            else:
                self._fused[tokens] = None
        return self._fused[tokens]

    def forward(self, x, B: int, pos: torch.Tensor):
        """``x [B*Tc/tp, D]`` (this rank's tokens) -> same shape.  ``pos [Tc]``: logical positions of the cp shard."""
        cfg, par = self.cfg, self.par
        tp, cp = par.tp, par.cp
        fused = self._fused_ops(x.shape[0] * tp.world) if (tp.world > 1 and _fast(x)) else None
        if fused is not None:
            from ..parallel.fused_linear import column_linear
            qkv = column_linear(x, self.w_qkv, fused[0])          # all-gather fused into the QKV GEMM
        else:
            xg = all_gather_seq(x, tp) if tp.world > 1 else x
            qkv = _linear(xg, self.w_qkv)
        Tc = qkv.shape[0] // B
        qkv = qkv.view(B, Tc, self.Hq + 2 * self.Hkv, self.hd)
        q, k, v = qkv[:, :, : self.Hq], qkv[:, :, self.Hq: self.Hq + self.Hkv], qkv[:, :, self.Hq + self.Hkv:]
        if _fast(x):
            from ..ops.attention import attention, ring_attention_autograd
            from ..ops.rope import rope
            cos, sin = self._tables(x.device)
            p32 = pos.to(torch.int32).repeat(B)
            q = rope(q.reshape(B * Tc, self.Hq, self.hd), p32, cos, sin).view(B, Tc, self.Hq, self.hd)
            k = rope(k.reshape(B * Tc, self.Hkv, self.hd), p32, cos, sin).view(B, Tc, self.Hkv, self.hd)
            v = v.contiguous()
            if cp.world > 1:
                o = ring_attention_autograd(q, k, v, cp.comm, causal=True, striped=cfg.striped)
            else:
                o = attention(q, k, v, causal=True)
        else:
            q, k = _rope_torch(q, pos, cfg.rope_theta), _rope_torch(k, pos, cfg.rope_theta)
            kpos = pos
            if cp.world > 1:
                k = _GatherKV.apply(k, cp.group, cp.world).transpose(0, 1).reshape(B, cp.world * Tc, self.Hkv, self.hd)
                v = _GatherKV.apply(v, cp.group, cp.world).transpose(0, 1).reshape(B, cp.world * Tc, self.Hkv, self.hd)
                kpos = torch.cat([shard_positions(cfg, cp.world, c, pos.device) for c in range(cp.world)])
            grp = self.Hq // self.Hkv
            kf, vf = k.repeat_interleave(grp, 2), v.repeat_interleave(grp, 2)
            s = torch.einsum("bthd,bshd->bhts", q, kf) * self.hd ** -0.5
            s = s.masked_fill((kpos[None, :] > pos[:, None])[None, None], float("-inf"))
            o = torch.einsum("bhts,bshd->bthd", torch.softmax(s.float(), -1).to(q.dtype), vf)
        if fused is not None:
            from ..parallel.fused_linear import row_linear
            return row_linear(o.reshape(B * Tc, self.Hq * self.hd), self.w_o, fused[1])   # GEMM -> reduce-scatter
        y = _linear(o.reshape(B * Tc, self.Hq * self.hd), self.w_o)
        return reduce_scatter_seq(y, tp) if tp.world > 1 else y


class Block(nn.Module):
    def __init__(self, cfg: HybridConfig, par: ParallelContext, layer: int, dtype, device, in_flight: int = 1):
        super().__init__()
        self.cfg = cfg
        self.norm1 = nn.Parameter(torch.ones(cfg.d_model, dtype=dtype, device=device))
        self.norm2 = nn.Parameter(torch.ones(cfg.d_model, dtype=dtype, device=device))
        self.attn = Attention(cfg, par, layer, dtype, device, in_flight)
        self.ffn = TPGatedFFN(cfg.d_model, cfg.d_ff, par.tp, cfg.act, sequence_parallel=True, dtype=dtype, device=device,
                              init_std=cfg.init_std, seed=2000 + layer, in_flight=in_flight)

    def forward(self, x, B, pos):
        x = x + self.attn(_norm(x, self.norm1, self.cfg.eps), B, pos)
        return x + self.ffn(_norm(x, self.norm2, self.cfg.eps))


def shard_positions(cfg: HybridConfig, cp_world: int, cp_rank: int, device) -> torch.Tensor:
    Tc = cfg.seq_len // cp_world
    if cfg.striped:
        return torch.arange(Tc, device=device) * cp_world + cp_rank
    return torch.arange(Tc, device=device) + cp_rank * Tc


class HybridStage(nn.Module):
    """The layers of one pipeline stage (plus the embedding on the first and the head on the last)."""

    def __init__(self, cfg: HybridConfig, par: ParallelContext, dtype=torch.bfloat16, device=None, in_flight: int = 1):
        super().__init__()
        self.cfg, self.par = cfg, par
        device = device or par.device
        self.layers_range = split_layers(cfg.n_layers, par.pp.world)[par.pp.rank]
        # in_flight: forward passes of this stage that can run before their backward passes (pipeline warm-up)
        self.blocks = nn.ModuleList(Block(cfg, par, i, dtype, device, in_flight) for i in self.layers_range)
        g = torch.Generator(device="cpu").manual_seed(7)
        emb = torch.empty(cfg.vocab, cfg.d_model).normal_(0, cfg.init_std, generator=g)
        head = torch.empty(cfg.vocab, cfg.d_model).normal_(0, cfg.init_std, generator=g)
        self.embed = nn.Parameter(emb.to(device=device, dtype=dtype)) if par.pp.first else None
        if par.pp.last:
            self.final_norm = nn.Parameter(torch.ones(cfg.d_model, dtype=dtype, device=device))
            self.head = nn.Parameter(head.to(device=device, dtype=dtype))
        self.pos = shard_positions(cfg, par.cp.world, par.cp.rank, device)
        for name, p in self.named_parameters():
            p.tp_sharded = ("w_qkv" in name) or ("w_o" in name) or ("w_gate_up" in name) or ("w_down" in name)

    # tokens of this rank: cp shard of every sample, then the tp slice of the flattened [B*Tc] tokens
    def local_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        """``tokens [B, T]`` (whole sequences of this data-parallel rank's samples) -> this rank's ``[B*Tc/tp]``."""
        tp = self.par.tp
        t = tokens[:, self.pos.to(tokens.device)].reshape(-1)
        n = t.numel() // tp.world
        return t[tp.rank * n:(tp.rank + 1) * n]

    def forward(self, x, B: int):
        if self.par.pp.first:
            x = F.embedding(x, self.embed)
        for blk in self.blocks:
            x = blk(x, B, self.pos)
        return x

    def loss(self, y, targets):
        """Sum of token cross-entropies of this rank's tokens divided by the number of tokens in the global batch
        (so that the sum over tp, cp and dp ranks is the mean loss)."""
        par, cfg = self.par, self.cfg
        h = _norm(y, self.final_norm, cfg.eps)
        logits = _linear(h, self.head).float()
        total = targets.numel() * par.tp.world * par.cp.world * par.dp.world
        return F.cross_entropy(logits, targets, reduction="sum") / total


class HybridTrainer:
    """One training step = pipeline schedule over the microbatches, gradient reduction over tp/cp/dp, AdamW."""

    def __init__(self, cfg: HybridConfig, par: ParallelContext, *, micro_batch: int = 1, n_micro: int = 2, lr: float = 1e-3,
                 dtype=torch.bfloat16):
        from ..parallel.optim import ShardedAdamW
        self.cfg, self.par, self.mb, self.M = cfg, par, micro_batch, n_micro
        self.stage = HybridStage(cfg, par, dtype=dtype, in_flight=max(1, min(n_micro, par.pp.world - par.pp.rank)))
        self.dtype = dtype
        self.params = [p for p in self.stage.parameters()]
        dp = par.dp
        self.opt = ShardedAdamW(self.params, lr=lr, dp_group=dp.group if dp.world > 1 else None, dp_world=dp.world,
                                dp_rank=dp.rank)
        tp, cp = par.tp, par.cp
        self.act_shape = (micro_batch * (cfg.seq_len // cp.world) // tp.world, cfg.d_model)

    def _sync_grads(self):
        """Replicated parameters saw only this rank's tokens: sum their gradients over tp; every parameter's over cp
        (the data-parallel average happens in the optimiser's reduce-scatter)."""
        par = self.par
        for axis, pick in ((par.tp, lambda p: not p.tp_sharded), (par.cp, lambda p: True)):
            if axis.world == 1:
                continue
            ps = [p for p in self.params if pick(p) and p.grad is not None]
            if not ps:
                continue
            flat = torch.cat([p.grad.reshape(-1).float() for p in ps])
            all_reduce_sum_(flat, axis)
            off = 0
            for p in ps:
                p.grad.copy_(flat[off: off + p.numel()].view_as(p))
                off += p.numel()

    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """``tokens, targets [n_micro * micro_batch, T]`` of this data-parallel rank (same on its tp/cp/pp ranks).
        Leaves in ``p.grad`` this rank's shard of the gradient of the global mean loss, summed over tp and cp and
        over this data-parallel rank's samples; returns the mean loss of the global batch (a 1-element tensor,
        valid on every rank)."""
        par, st = self.par, self.stage
        B = self.mb
        micro_in = [st.local_tokens(tokens[i * B:(i + 1) * B]) for i in range(self.M)]
        micro_tg = [st.local_tokens(targets[i * B:(i + 1) * B]) for i in range(self.M)]
        for p in self.params:
            p.grad = None
        # the loss of a microbatch is already divided by its global token count; average over the microbatches
        losses, self.stats = run_1f1b(lambda x: st(x, B), par.pp, micro_in, act_shape=self.act_shape, act_dtype=self.dtype,
                                      loss_fn=st.loss if par.pp.last else None, targets=micro_tg, grad_scale=1.0 / self.M)
        self._sync_grads()
        for p in self.params:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
        loss = torch.stack(losses).sum() / self.M if losses else torch.zeros((), device=par.device)
        loss = loss.float().reshape(1)
        if par.world > 1 and dist.is_initialized():
            dist.all_reduce(loss)                      # sums the tp/cp/dp parts on the last stage; zeros elsewhere
        return loss

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimiser step; returns the loss tensor of :meth:`forward_backward` (no host synchronisation)."""
        loss = self.forward_backward(tokens, targets)
        # data-parallel ranks hold different samples and the loss is already normalised by the global batch: the
        # gradient is the SUM over dp, while the optimiser's reduce-scatter averages; undo its division
        if self.par.dp.world > 1:
            for p in self.params:
                p.grad.mul_(self.par.dp.world)
        self.opt.step()
        return loss


def all_reduce_sum_(flat: torch.Tensor, axis) -> None:
    from ..parallel.collectives_autograd import _ar
    _ar(flat, axis)


def reference_loss_and_grads(cfg: HybridConfig, tokens, targets, dtype=torch.float32, device="cpu"):
    """The same model on one process (grid 1x1x1x1): mean loss and the full gradients by parameter name."""
    par = ParallelContext(None, ParallelDims())
    st = HybridStage(cfg, par, dtype=dtype, device=torch.device(device))
    B = tokens.shape[0]
    y = st(st.local_tokens(tokens), B)
    loss = st.loss(y, st.local_tokens(targets))
    loss.backward()
    return float(loss), {n: p.grad for n, p in st.named_parameters()}, st
