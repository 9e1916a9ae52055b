"""Routed MoE layer, expert parallel over all ranks, training forward + backward.

d_model 2048, 64 SwiGLU experts of d_ff 1408, softmax router top-6, 8192 tokens per rank, a per-rank expert bias
~ N(0,1) on the logits so that loads are skewed and uneven; bf16.

``--impl mesh``: fused dispatch / grouped tcgen05 GEMMs / combine over peer memory (``mesh_b200/parallel/moe.py``).
``--impl baseline``: the same layer in stock PyTorch: sort by expert, ``all_to_all_single`` over NCCL for counts and
rows, a loop of cuBLAS matmuls over the local experts, all-to-all back, autograd for the backward.
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist
import torch.nn.functional as F

from common import emit, init, time_steps


def baseline_layer(x, w_router, w1, w2, bias, k, E, world, group):
    """x [T, D] -> [T, D]; w1 [El, 2F, D], w2 [El, D, F] (requires_grad leaves)."""
    from torch.distributed.nn.functional import all_to_all_single
    T, D = x.shape
    El = E // world
    logits = (x @ w_router.T).float() + bias
    p = torch.softmax(logits, -1)
    w, idx = torch.topk(p, k, -1)
    w = (w / w.sum(-1, keepdim=True)).to(x.dtype)
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    rows = x[order // k]
    counts = torch.bincount(flat, minlength=E)
    if world > 1:
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=group)          # [world, El] counts from every source
        send_splits = counts.view(world, El).sum(1).tolist()
        recv_splits = recv_counts.view(world, El).sum(1).tolist()
        got = all_to_all_single(rows.new_empty((sum(recv_splits), D)), rows, recv_splits, send_splits, group=group)
        # rows arrive grouped by source, then by expert: regroup by expert
        rc = recv_counts.view(world, El)
        eid = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(world), rc.reshape(-1))
        perm = torch.argsort(eid, stable=True)
        xin = got[perm]
        per_expert = rc.sum(0).tolist()
    else:
        xin, per_expert, perm = rows, counts.tolist(), None
    outs = []
    Fh = w1.shape[1] // 2
    lo = 0
    for e in range(El):
        n = per_expert[e]
        xe = xin[lo: lo + n]
        h = F.silu(xe @ w1[e, :Fh].T) * (xe @ w1[e, Fh:].T)
        outs.append(h @ w2[e].T)
        lo += n
    y = torch.cat(outs)
    if world > 1:
        back = torch.empty_like(y)
        back[perm] = y
        y = all_to_all_single(y.new_empty((sum(send_splits), D)), back, send_splits, recv_splits, group=group)
    out = torch.zeros_like(x)
    out.index_add_(0, order // k, y * w.reshape(-1)[order][:, None])
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="mesh", choices=["mesh", "baseline"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--d-ff", type=int, default=1408)
    ap.add_argument("--top-k", type=int, default=6)
    ap.add_argument("--phases", action="store_true", help="mesh arm: also report the time of every phase of a step")
    a = ap.parse_args()
    from mesh_b200.config import MeshConfig, set_config
    set_config(MeshConfig.from_env(heap_bytes=8 << 30))
    ctx = init()
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    T, D, Fh, E, k = a.tokens, a.d_model, a.d_ff, a.experts, a.top_k
    El = E // world
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    x = torch.randn(T, D, generator=g).bfloat16().to(dev)
    dy = torch.randn(T, D, generator=g).bfloat16().to(dev)
    bias = torch.randn(E, generator=g).to(dev)
    gw = torch.Generator(device="cpu").manual_seed(7)
    w_router = torch.empty(E, D).normal_(0, 0.02, generator=gw).bfloat16().to(dev)
    w1 = torch.empty(E, 2 * Fh, D).normal_(0, 0.02, generator=gw)[rank * El:(rank + 1) * El].bfloat16().to(dev)
    w2 = torch.empty(E, D, Fh).normal_(0, 0.02, generator=gw)[rank * El:(rank + 1) * El].bfloat16().to(dev)
    launches = 0
    if a.impl == "mesh":
        from mesh_b200 import _native
        from mesh_b200.parallel.moe import EPMoE
        from mesh_b200.utils.status import check_status
        moe = EPMoE(ctx, T, D, Fh, E, k)
        w1f, w2f = w1.reshape(El * 2 * Fh, D).contiguous(), w2.reshape(El * D, Fh).contiguous()

        def step():
            moe.forward(x, w_router, w1f, w2f, bias)
            moe.backward(dy)
        l0 = _native.launch_count
        step()
        launches = _native.launch_count - l0
    else:
        wr = w_router.clone().requires_grad_(True)
        w1p, w2p = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
        xp = x.clone().requires_grad_(True)
        grp = ctx.group if world > 1 else None

        def step():
            for t in (wr, w1p, w2p, xp):
                t.grad = None
            baseline_layer(xp, wr, w1p, w2p, bias, k, E, world, grp).backward(dy)
    ms = time_steps(step, a.steps, a.warmup, world, dev)
    phases = None
    if a.impl == "mesh":
        check_status()
        if a.phases:
            import statistics
            per: dict = {}
            for _ in range(5):
                moe.timeline = []
                step()
                torch.cuda.synchronize()
                for name, us in moe.phases(moe.timeline):
                    per.setdefault(name, []).append(us)
            moe.timeline = None
            phases = {name: round(statistics.median(v), 1) for name, v in per.items()}
    flops = 3 * T * k * (2 * D * 2 * Fh + 2 * Fh * D) * world
    emit(rank, {"metric": "moe_ep_train_tokens_per_s", "value": round(T * world / (ms * 1e-3), 1), "unit": "tokens/s (fwd+bwd)",
                "impl": a.impl, "n_gpus": world, "ms_per_step": round(ms, 4), "steps": a.steps,
                "tflops_total": round(flops / (ms * 1e-3) / 1e12, 1), "gpu_launches_per_step": launches,
                **({"phase_us_rank0": phases} if phases else {}),
                "config": {"tokens_per_rank": T, "d_model": D, "experts": E, "d_ff": Fh, "top_k": k, "ep": world,
                           "skew": "per-rank N(0,1) expert bias", "l2": "256 MiB flush write between steps (untimed)"}})
    from mesh_b200.distributed import shutdown
    shutdown()


if __name__ == "__main__":
    main()
