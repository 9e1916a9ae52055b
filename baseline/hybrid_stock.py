"""Stock arm of the hybrid training benchmark: the same decoder and the same tp x cp x pp x dp grid, built from what
PyTorch ships and nothing of this package.

* tensor parallel: the Megatron recipe with ``torch.distributed`` collectives - column-parallel ``F.linear``, the
  row-parallel one followed by an all-reduce (identity / all-reduce pairs as autograd functions);
* context parallel: contiguous token blocks, keys and values all-gathered over the axis (reduce-scatter backward),
  ``F.scaled_dot_product_attention`` with a boolean mask for the block's rows;
* pipeline: all microbatches forward, then all backward, activations passed with ``dist.send`` / ``dist.recv``;
* data parallel: gradients all-reduced after the backward pass; ``torch.optim.AdamW`` (fused on CUDA).

Runs under NCCL on GPUs and under gloo on CPU ranks (fp32), which is how its sharding is tested against its own
single-process run.  ``python benchmarks/hybrid_step.py --impl stock`` times it with the same clock as the other arm.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class StockConfig:
    vocab: int = 4096
    d_model: int = 1024
    n_layers: int = 4
    n_heads: int = 8
    n_kv_heads: int = 8
    head_dim: int = 128
    d_ff: int = 4096
    seq_len: int = 1024
    rope_theta: float = 10000.0
    eps: float = 1e-6
    init_std: float = 0.02


class Grid:
    """Rank arithmetic and process groups of a (dp, pp, cp, tp) grid, tp fastest."""

    def __init__(self, text: str, rank: int, world: int):
        found = {k: int(v) for k, v in re.findall(r"(dp|pp|cp|tp)\s*=?\s*(\d+)", text.lower())}
        self.size = {ax: found.get(ax, 1) for ax in ("dp", "pp", "cp", "tp")}
        if math.prod(self.size.values()) != world:
            raise ValueError(f"grid {text!r} needs {math.prod(self.size.values())} ranks, the job has {world}")
        self.rank, self.world = rank, world
        self.coord, rest = {}, rank
        for ax in ("tp", "cp", "pp", "dp"):
            self.coord[ax], rest = rest % self.size[ax], rest // self.size[ax]
        self.groups, self.members = {}, {}
        stride = 1
        for ax in ("tp", "cp", "pp", "dp"):
            n = self.size[ax]
            for base in range(world):
                if (base // stride) % n:
                    continue                                   # not the first member of its line
                line = [base + i * stride for i in range(n)]
                group = dist.new_group(line) if (n > 1 and world > 1) else None      # every rank creates every group
                if rank in line:
                    self.groups[ax], self.members[ax] = group, line
            stride *= n


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherTokens(torch.autograd.Function):
    """All-gather along the token dimension (dim 2 of ``[B, H, T, hd]``); the backward sums and keeps this block."""

    @staticmethod
    def forward(ctx, x, group, world, index):
        ctx.group, ctx.world, ctx.index = group, world, index
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, 2)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g.chunk(ctx.world, 2)[ctx.index].contiguous(), None, None, None


def _rms(x, w, eps):
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def _rope(x, pos, theta):
    """``x [B, H, T, hd]``, rotate-half."""
    hd = x.shape[-1]
    inv = theta ** (-torch.arange(0, hd, 2, device=x.device, dtype=torch.float32) / hd)
    ang = pos.float()[:, None] * inv[None]
    cos, sin = ang.cos()[None, None], ang.sin()[None, None]
    x1, x2 = x[..., : hd // 2].float(), x[..., hd // 2:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


class Block(nn.Module):
    def __init__(self, cfg: StockConfig, grid: Grid, layer: int, dtype, device):
        super().__init__()
        self.cfg, self.grid = cfg, grid
        tp, r = grid.size["tp"], grid.coord["tp"]
        assert cfg.n_heads % tp == 0 and cfg.n_kv_heads % tp == 0 and cfg.d_ff % tp == 0
        self.Hq, self.Hkv, hd, D, Fh = cfg.n_heads // tp, cfg.n_kv_heads // tp, cfg.head_dim, cfg.d_model, cfg.d_ff // tp
        g = torch.Generator(device="cpu").manual_seed(1000 + layer)
        full = lambda rows, cols, std: torch.empty(rows, cols).normal_(0, std, generator=g)
        out_std = cfg.init_std / math.sqrt(2 * cfg.n_layers)
        wq, wk, wv = full(cfg.n_heads * hd, D, cfg.init_std), full(cfg.n_kv_heads * hd, D, cfg.init_std), full(cfg.n_kv_heads * hd, D, cfg.init_std)
        wo = full(D, cfg.n_heads * hd, out_std)
        w1, w3, w2 = full(cfg.d_ff, D, cfg.init_std), full(cfg.d_ff, D, cfg.init_std), full(D, cfg.d_ff, out_std)
        qs, ks, fs = slice(r * self.Hq * hd, (r + 1) * self.Hq * hd), slice(r * self.Hkv * hd, (r + 1) * self.Hkv * hd), slice(r * Fh, (r + 1) * Fh)
        put = lambda t: nn.Parameter(t.contiguous().to(device=device, dtype=dtype))
        self.w_qkv, self.w_o = put(torch.cat([wq[qs], wk[ks], wv[ks]], 0)), put(wo[:, qs])
        self.w_13, self.w_2 = put(torch.cat([w1[fs], w3[fs]], 0)), put(w2[:, fs])
        self.n1, self.n2 = put(torch.ones(D)), put(torch.ones(D))

    def forward(self, x, pos, mask):
        cfg, grid = self.cfg, self.grid
        B, T, D = x.shape
        tp_group, cp = grid.groups.get("tp"), grid.size["cp"]
        tp_on = grid.size["tp"] > 1
        h = _rms(x, self.n1, cfg.eps)
        if tp_on:
            h = _CopyToTP.apply(h, tp_group)
        qkv = F.linear(h, self.w_qkv)
        hd = cfg.head_dim
        q, k, v = qkv.split([self.Hq * hd, self.Hkv * hd, self.Hkv * hd], -1)
        q = _rope(q.view(B, T, self.Hq, hd).transpose(1, 2), pos, cfg.rope_theta)
        k = _rope(k.view(B, T, self.Hkv, hd).transpose(1, 2), pos, cfg.rope_theta)
        v = v.view(B, T, self.Hkv, hd).transpose(1, 2)
        if cp > 1:
            k = _GatherTokens.apply(k, grid.groups["cp"], cp, grid.coord["cp"])
            v = _GatherTokens.apply(v, grid.groups["cp"], cp, grid.coord["cp"])
        if self.Hkv != self.Hq:
            k, v = (t.repeat_interleave(self.Hq // self.Hkv, 1) for t in (k, v))
        if mask is None:
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        else:
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        o = F.linear(a.transpose(1, 2).reshape(B, T, self.Hq * hd), self.w_o)
        if tp_on:
            o = _ReduceFromTP.apply(o, tp_group)
        x = x + o
        h = _rms(x, self.n2, cfg.eps)
        if tp_on:
            h = _CopyToTP.apply(h, tp_group)
        gate, up = F.linear(h, self.w_13).chunk(2, -1)
        y = F.linear(F.silu(gate) * up, self.w_2)
        if tp_on:
            y = _ReduceFromTP.apply(y, tp_group)
        return x + y


class Stage(nn.Module):
    """The layers of one pipeline stage; the first stage embeds, the last one normalises, projects and scores."""

    def __init__(self, cfg: StockConfig, grid: Grid, dtype, device):
        super().__init__()
        self.cfg, self.grid = cfg, grid
        pp, s = grid.size["pp"], grid.coord["pp"]
        per = -(-cfg.n_layers // pp)
        self.first, self.last = s == 0, s == pp - 1
        self.blocks = nn.ModuleList(Block(cfg, grid, l, dtype, device) for l in range(s * per, min(cfg.n_layers, (s + 1) * per)))
        g = torch.Generator(device="cpu").manual_seed(7)
        emb = torch.empty(cfg.vocab, cfg.d_model).normal_(0, cfg.init_std, generator=g)
        head = torch.empty(cfg.vocab, cfg.d_model).normal_(0, cfg.init_std, generator=g)
        if self.first:
            self.embed = nn.Parameter(emb.to(device=device, dtype=dtype))
        if self.last:
            self.norm = nn.Parameter(torch.ones(cfg.d_model, device=device, dtype=dtype))
            self.head = nn.Parameter(head.to(device=device, dtype=dtype))
        cp, c = grid.size["cp"], grid.coord["cp"]
        Tc = cfg.seq_len // cp
        self.pos = torch.arange(c * Tc, (c + 1) * Tc, device=device)
        self.mask = None
        if cp > 1:                                            # this block's rows of the causal mask over all keys
            self.mask = self.pos[:, None] >= torch.arange(cfg.seq_len, device=device)[None, :]

    def forward(self, x_or_tokens, targets=None):
        x = F.embedding(x_or_tokens, self.embed) if self.first else x_or_tokens
        for b in self.blocks:
            x = b(x, self.pos, self.mask)
        if not self.last:
            return x
        logits = F.linear(_rms(x, self.norm, self.cfg.eps), self.head).float()
        return F.cross_entropy(logits.view(-1, logits.shape[-1]), targets.reshape(-1), reduction="sum")


class StockTrainer:
    """One optimiser step over ``n_micro`` microbatches of ``[micro_batch, seq_len]`` token ids per data-parallel rank."""

    def __init__(self, cfg: StockConfig, grid: Grid, device, dtype, micro_batch: int = 1, n_micro: int = 1, lr: float = 1e-4):
        self.cfg, self.grid, self.device, self.dtype = cfg, grid, device, dtype
        self.B, self.M = micro_batch, n_micro
        if cfg.seq_len % grid.size["cp"]:
            raise ValueError("the sequence must divide over the context axis")
        self.stage = Stage(cfg, grid, dtype, device)
        self.params = [p for p in self.stage.parameters()]
        self.opt = torch.optim.AdamW(self.params, lr=lr, betas=(0.9, 0.95), weight_decay=0.0, fused=device.type == "cuda")
        line = grid.members.get("pp", [grid.rank])
        s = grid.coord["pp"]
        self.prev = line[s - 1] if s > 0 else None
        self.next = line[s + 1] if s + 1 < len(line) else None
        self.Tc = cfg.seq_len // grid.size["cp"]

    def _local(self, ids):
        c = self.grid.coord["cp"]
        return ids[:, c * self.Tc:(c + 1) * self.Tc]

    def forward_backward(self, tokens, targets):
        """``tokens, targets [n_micro * micro_batch, seq_len]`` on the device -> the mean loss (valid on the last stage;
        all-reduced over the grid so every rank returns it)."""
        st, B, M = self.stage, self.B, self.M
        scale = 1.0 / (M * B * self.cfg.seq_len)
        shape = (B, self.Tc, self.cfg.d_model)
        kept, total = [], torch.zeros((), device=self.device, dtype=torch.float32)
        for m in range(M):
            sl = slice(m * B, (m + 1) * B)
            if st.first:
                inp = self._local(tokens[sl])
            else:
                inp = torch.empty(shape, device=self.device, dtype=self.dtype)
                dist.recv(inp, src=self.prev)
                inp.requires_grad_(True)
            out = st(inp, self._local(targets[sl]) if st.last else None)
            if st.last:
                total += out.detach()
            else:
                dist.send(out.detach().contiguous(), dst=self.next)
            kept.append((inp, out))
        for m in range(M):
            inp, out = kept[m]
            if st.last:
                (out * scale).backward()
            else:
                g = torch.empty(shape, device=self.device, dtype=self.dtype)
                dist.recv(g, src=self.next)
                out.backward(g)
            if not st.first:
                dist.send(inp.grad.contiguous(), dst=self.prev)
            kept[m] = None
        for ax in ("cp", "dp"):
            n = self.grid.size[ax]
            if n > 1:
                for p in self.params:
                    if p.grad is not None:
                        dist.all_reduce(p.grad, group=self.grid.groups[ax])
                        if ax == "dp":
                            p.grad.div_(n)
        loss = total * scale
        if self.grid.world > 1:
            if not st.last or self.grid.coord["tp"] != 0:
                loss = torch.zeros_like(loss)                  # one copy of every token's loss enters the sum
            dist.all_reduce(loss)
            loss = loss / self.grid.size["dp"]
        return loss

    def step(self, tokens, targets):
        self.opt.zero_grad(set_to_none=True)
        loss = self.forward_backward(tokens, targets)
        self.opt.step()
        return loss
