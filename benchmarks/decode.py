"""E2B-class decoder inference: greedy decode tokens/s at TP = world size, bf16 and 4-bit group-64 weights,
batch 1 and 8, prompt 512, 256 decode steps.

``--impl mesh``: this package's decode kernels under one CUDA graph (``mesh_b200/models/e2b.py``).
``--impl baseline``: the same architecture in stock PyTorch: cuBLAS linears, ``scaled_dot_product_attention`` over
a static KV cache, NCCL all-reduce after the two row-parallel projections, vocab-parallel logits all-gathered for the
argmax; the decode step is captured in a CUDA graph as well, so both arms replay one graph per token.  The baseline
has bf16 weights only (stock PyTorch has no 4-bit group-quantised matmul).
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist
import torch.nn.functional as F

from common import emit, init


class BaselineDecoder:
    def __init__(self, cfg, rank, world, group, B, dev):
        self.cfg, self.rank, self.world, self.group, self.B, self.dev = cfg, rank, world, group, B, dev
        c = cfg
        self.Hq, self.Hkv, hd = c.q_heads // world, max(1, c.kv_heads // world), c.head_dim
        Fl = c.d_ff // world
        gen = torch.Generator(device=dev).manual_seed(1)

        def w(*shape):
            return (torch.randn(shape, generator=gen, device=dev) * c.init_std).to(torch.bfloat16)
        self.layers = []
        for _ in range(c.layers):
            self.layers.append(dict(n1=torch.ones(c.d_model, device=dev, dtype=torch.bfloat16), n2=torch.ones(c.d_model, device=dev, dtype=torch.bfloat16),
                                    qkv=w((self.Hq + 2 * self.Hkv) * hd, c.d_model), o=w(c.d_model, self.Hq * hd),
                                    gu=w(2 * Fl, c.d_model), down=w(c.d_model, Fl),
                                    k=torch.zeros(B, self.Hkv, c.max_seq, hd, device=dev, dtype=torch.bfloat16),
                                    v=torch.zeros(B, self.Hkv, c.max_seq, hd, device=dev, dtype=torch.bfloat16)))
        self.embed = w(c.vocab // world, c.d_model)           # tied: vocab-parallel rows
        self.fn = torch.ones(c.d_model, device=dev, dtype=torch.bfloat16)
        inv = 1.0 / (c.theta ** (torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd))
        ang = torch.arange(c.max_seq, device=dev, dtype=torch.float32)[:, None] * inv[None]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.pos = torch.zeros((), dtype=torch.long, device=dev)
        self.tok = torch.zeros(B, dtype=torch.long, device=dev)
        self.span = torch.arange(c.max_seq, device=dev)

    def _norm(self, x, w):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.cfg.eps)).to(x.dtype) * w

    def _rope(self, x, pos):
        hd = x.shape[-1]
        idx = pos.reshape(1)                                  # a device scalar: no host read inside the captured step
        cos, sin = self.cos.index_select(0, idx)[None], self.sin.index_select(0, idx)[None]
        x1, x2 = x[..., : hd // 2].float(), x[..., hd // 2:].float()
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)

    def _embed(self, tok):
        V = self.cfg.vocab // self.world
        local = tok - self.rank * V
        ok = (local >= 0) & (local < V)
        x = F.embedding(local.clamp(0, V - 1), self.embed) * ok[:, None].to(torch.bfloat16)
        if self.world > 1:
            dist.all_reduce(x, group=self.group)
        return x

    def step(self):
        """One token for every sequence of the batch at position ``self.pos`` (a device scalar)."""
        c, B = self.cfg, self.B
        x = self._embed(self.tok)
        pos = self.pos
        for i, L in enumerate(self.layers):
            h = self._norm(x, L["n1"])
            qkv = F.linear(h, L["qkv"]).view(B, self.Hq + 2 * self.Hkv, c.head_dim)
            q, k, v = qkv[:, : self.Hq], qkv[:, self.Hq: self.Hq + self.Hkv], qkv[:, self.Hq + self.Hkv:]
            q, k = self._rope(q, pos), self._rope(k, pos)
            L["k"].index_copy_(2, pos.reshape(1), k[:, :, None])
            L["v"].index_copy_(2, pos.reshape(1), v[:, :, None])
            vis = self.span <= pos
            if c.is_local(i):
                vis = vis & (self.span > pos - c.window)
            o = F.scaled_dot_product_attention(q[:, :, None], L["k"], L["v"], attn_mask=vis[None, None, None, :], enable_gqa=True)
            y = F.linear(o.reshape(B, self.Hq * c.head_dim), L["o"])
            if self.world > 1:
                dist.all_reduce(y, group=self.group)
            x = x + y
            h = self._norm(x, L["n2"])
            gu = F.linear(h, L["gu"])
            Fl = gu.shape[1] // 2
            y = F.linear(F.gelu(gu[:, :Fl], approximate="tanh") * gu[:, Fl:], L["down"])
            if self.world > 1:
                dist.all_reduce(y, group=self.group)
            x = x + y
        logits = F.linear(self._norm(x, self.fn), self.embed).float()
        if self.world > 1:
            full = torch.empty(self.world, B, logits.shape[1], device=self.dev)
            dist.all_gather_into_tensor(full, logits.contiguous(), group=self.group)
            logits = full.permute(1, 0, 2).reshape(B, -1)
        self.tok.copy_(logits.argmax(-1))
        self.pos.add_(1)


def run_baseline(ctx, cfg, B, prompt_len, steps):
    m = BaselineDecoder(cfg, ctx.rank, ctx.world, ctx.group if ctx.world > 1 else None, B, ctx.device)
    # the prompt is fed token by token through the same step (the timed region is the decode only)
    g = torch.Generator(device="cpu").manual_seed(11)
    prompt = torch.randint(0, cfg.vocab, (B, prompt_len), generator=g).to(ctx.device)
    with torch.no_grad():
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                m.step()
        torch.cuda.current_stream().wait_stream(side)
        m.pos.zero_()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):   # the runtime's monitor thread is running
            m.step()
        m.pos.zero_()
        for t in range(prompt_len):
            m.tok.copy_(prompt[:, t])
            graph.replay()
        torch.cuda.synchronize()
        if ctx.world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=ctx.device, dtype=torch.float64)
    if ctx.world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms[0])


def explain_baseline(ctx, cfg, B: int = 1) -> dict:
    """Kernels of one eager step of the stock decoder: how many, their summed device time, and the largest groups."""
    from torch.profiler import ProfilerActivity, profile
    m = BaselineDecoder(cfg, ctx.rank, ctx.world, ctx.group if ctx.world > 1 else None, B, ctx.device)
    with torch.no_grad():
        for _ in range(3):
            m.step()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            m.step()
            torch.cuda.synchronize()
    rows = [(e.key, e.count, e.device_time_total) for e in prof.key_averages() if e.device_time_total > 0]
    rows.sort(key=lambda r: -r[2])
    return {"kernels": int(sum(r[1] for r in rows)), "device_us": round(sum(r[2] for r in rows), 1),
            "top": [{"kernel": k[:60], "launches": int(n), "us": round(t, 1)} for k, n, t in rows[:8]]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="mesh", choices=["mesh", "baseline"])
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--explain", action="store_true",
                    help="baseline arm: where a decode step's time goes (kernels of one eager step by device time)")
    a = ap.parse_args()
    ctx = init()
    from mesh_b200.models.e2b import E2BConfig, bench_decode
    cfg = E2BConfig()
    if a.impl == "mesh":
        rec = bench_decode(ctx, steps=a.steps, prompt_len=a.prompt)
        from mesh_b200.utils.status import check_status
        check_status()
    else:
        rec = {"model": "E2B-class decoder (30L, d2048, 8q/2kv x256, GeGLU 8192, SWA 512 4:1, vocab 262144 tied)",
               "prompt": a.prompt, "decode_steps": a.steps, "tp": ctx.world, "runs": []}
        for B in (1, 8):
            ms = run_baseline(ctx, cfg, B, a.prompt, a.steps)
            rec["runs"].append({"weights": "bf16", "batch": B, "ms_per_token": round(ms / a.steps, 4),
                                "tokens_per_s": round(B * a.steps / (ms * 1e-3), 1)})
            torch.cuda.empty_cache()
        if a.explain:
            rec["baseline_step_kernels"] = explain_baseline(ctx, cfg)
    rec.update({"metric": "e2b_decode_tokens_per_s", "impl": a.impl, "n_gpus": ctx.world})
    emit(ctx.rank, rec)
    from mesh_b200.distributed import shutdown
    shutdown()


if __name__ == "__main__":
    main()
