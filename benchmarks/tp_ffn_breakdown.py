#!/usr/bin/env python
"""Per-kernel breakdown of the tensor-parallel FFN step (x[4096,4096], d_ff 14336, bf16) at N GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29517 \
        benchmarks/tp_ffn_breakdown.py

Prints one JSON line: the six launches of a layer (forward + backward) timed one by one with CUDA events (launches
serialised, ``MESH_GEMM_CHAIN=0`` semantics), the same six GEMMs run locally with no communication, the step with the
launches chained (the default), the stock PyTorch + NCCL + cuBLAS arm, and the bytes each fused kernel sends over
NVLink with the time those bytes need at the measured peer bandwidth.  Every number is the median over the timed
steps and the maximum over ranks.

``--shard-of N`` on one GPU times the local GEMMs at the shard shapes of an N-GPU job (d_ff / N columns): what the
tensor cores of one rank need at that N, tile waves included, with no GPU but this one.
"""
from __future__ import annotations

import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

TOKENS, D_MODEL, D_FF = 4096, 4096, 14336
PEER_GBS = 770.0           # measured peer copy bandwidth per direction per GPU on this pool
STEPS, WARMUP = 30, 5


def main() -> int:
    from mesh_b200.distributed import init, shutdown
    from mesh_b200.ops import gemm as G
    from mesh_b200.parallel.tp_ffn import FusedTPFFN
    from mesh_b200.utils.status import check_status
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--shard-of", type=int, default=0)
    a = ap.parse_args()
    ctx = init(backend="nccl")
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    shard_of = a.shard_of if (a.shard_of and world == 1) else world
    rows, Fl = TOKENS // world, D_FF // shard_of
    g = torch.Generator(device="cpu").manual_seed(1)
    x = torch.randn(rows, D_MODEL, generator=g).bfloat16().to(dev)
    dy = torch.randn(rows, D_MODEL, generator=g).bfloat16().to(dev)
    wgu = (torch.randn(2 * Fl, D_MODEL, generator=g) * 0.02).bfloat16().to(dev)
    wd = (torch.randn(D_MODEL, Fl, generator=g) * 0.02).bfloat16().to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def maxr(v):
        t = torch.tensor(v, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [round(float(a), 1) for a in t]

    def step_time(fn):
        for _ in range(WARMUP):
            fn()
        ts = []
        for _ in range(STEPS):
            flush.zero_()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    out = {"n_gpus": world, "shard_of": shard_of, "tokens": TOKENS, "d_model": D_MODEL, "d_ff": D_FF}
    if world > 1:
        op = FusedTPFFN(ctx.heap, TOKENS, D_MODEL, D_FF)

        def fused():
            op.forward(x, wgu, wd)
            op.backward(dy)

        op.chain = True
        out["fused_chained_us"] = maxr([step_time(fused)])[0]
        op.chain = False
        out["fused_serial_us"] = maxr([step_time(fused)])[0]
        per: dict[str, list] = {}
        order: list[str] = []
        for i in range(WARMUP + STEPS):
            flush.zero_()
            dist.barrier()
            with G.trace() as t:
                fused()
            if i >= WARMUP:
                for j, (label, us) in enumerate(t.report()):
                    key = f"{j + 1}:{label}"
                    per.setdefault(key, []).append(us)
                    if key not in order:
                        order.append(key)
        med = maxr([statistics.median(per[k]) for k in order])
        out["fused_kernels_us"] = dict(zip(order, med))
        op.chain = True
        check_status()

    # the same six GEMMs with every operand local (no gather, no scatter): what the tensor cores need
    X = torch.randn(TOKENS, D_MODEL, device=dev).bfloat16()
    DY = torch.randn(TOKENS, D_MODEL, device=dev).bfloat16()
    names = ["1:glu_fwd", "2:down", "3:glu_bwd", "4:dWd", "5:dx", "6:dWgu"]
    per = {n: [] for n in names}
    for i in range(WARMUP + STEPS):
        flush.zero_()
        with G.trace() as t:
            h, gu = G.glu_fwd(X, wgu)
            G.gemm(h, wd)
            dgu = G.glu_bwd(DY, wd, gu)
            G.gemm(DY, h, a_mn=True, b_mn=True)
            G.gemm(dgu, wgu, b_mn=True)
            G.gemm(dgu, X, a_mn=True, b_mn=True)
        if i >= WARMUP:
            for n, (_, us) in zip(names, t.report()):
                per[n].append(us)
    out["local_gemms_us"] = dict(zip(names, maxr([statistics.median(per[n]) for n in names])))
    out["local_gemms_sum_us"] = round(sum(out["local_gemms_us"].values()), 1)

    # stock arm
    from baseline.tp_ffn import tp_ffn
    wg_s, wu_s = wgu[:Fl].clone().requires_grad_(True), wgu[Fl:].clone().requires_grad_(True)
    wd_s = wd.clone().requires_grad_(True)
    xs = x.clone().requires_grad_(True)
    grp = ctx.group if world > 1 else None

    def stock():
        wg_s.grad = wu_s.grad = wd_s.grad = xs.grad = None
        tp_ffn(xs, wg_s, wu_s, wd_s, grp).backward(dy)

    out["stock_us"] = maxr([step_time(stock)])[0]

    # NVLink bytes per rank and the time they need at the measured peer bandwidth
    remote = (world - 1) / world
    ag_bytes = rows * D_MODEL * 2 * (world - 1)                 # this rank's shard stored into every peer
    rs_bytes = TOKENS * D_MODEL * 2 * remote                    # partial tiles stored to their owners
    flops = 3 * (2 * TOKENS * D_MODEL * 2 * D_FF + 2 * TOKENS * D_FF * D_MODEL) / shard_of
    from mesh_b200.config import capacity
    peak = capacity().get("bf16_tflops_sustained", 1382.0)
    out["link"] = {"all_gather_bytes_per_launch": int(ag_bytes), "reduce_scatter_bytes_per_launch": int(rs_bytes),
                   "all_gather_us_at_770GBs": round(ag_bytes / PEER_GBS / 1e3, 1),
                   "reduce_scatter_us_at_770GBs": round(rs_bytes / PEER_GBS / 1e3, 1),
                   "step_flops_per_gpu": flops, "step_us_at_measured_sustained_peak": round(flops / peak / 1e6, 1)}
    if rank == 0:
        print(json.dumps(out), flush=True)
    shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
