"""Small single-GPU workloads for profiler captures (one op per invocation, a few launches).

    python -m mesh_b200.tools.prof_ops gemm --m 4096 --n 4096 --k 4096 --iters 3
    python -m mesh_b200.tools.prof_ops glu_fwd | glu_bwd | rmsnorm | rope | router
    python -m mesh_b200.tools.prof_ops flash_fwd | flash_bwd --m <seq> --n <heads> --k <head_dim> [--time]
    python -m mesh_b200.tools.prof_ops decode_linear --m <batch> --n <out rows> --k <in cols> [--time]
    python -m mesh_b200.tools.prof_ops e2b_decode --m <batch> [--n 4] [--k <position>]    (the last step is bracketed
                                       with cudaProfilerStart/Stop for `ncu --profile-from-start off`)
    python -m mesh_b200.tools.prof_ops e2b_step_timeline --m <batch> [--n 4|8]             (step kernel, per-operation times)

Sizes are chosen larger than L2 (126 MB) in total footprint where DRAM figures matter but a few
hundred MB at most, so a full-metric capture of one or two launches ends by itself in about a minute.
"""
from __future__ import annotations

import argparse

import torch


def _time(run, flops, what, bytes_moved=0, iters=20):
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    extra = f" {flops / ms / 1e9:.1f} TFLOP/s" if flops else ""
    extra += f" {bytes_moved / ms / 1e6:.1f} GB/s" if bytes_moved else ""
    print(f"{what}: {ms * 1e3:.1f} us{extra}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("op")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--time", action="store_true", help="also print a CUDA-event timing of the op (not under a profiler)")
    a = ap.parse_args()
    from mesh_b200.ops import gemm as G
    from mesh_b200.utils.status import check_status
    dev = "cuda"
    torch.manual_seed(0)
    if a.op == "gemm":
        x = torch.randn(a.m, a.k, device=dev).bfloat16()
        w = torch.randn(a.n, a.k, device=dev).bfloat16()
        for _ in range(a.iters):
            G.gemm(x, w)
    elif a.op == "glu_fwd":
        x = torch.randn(a.m, a.k, device=dev).bfloat16()
        w = (torch.randn(2 * a.n, a.k, device=dev) * 0.02).bfloat16()
        for _ in range(a.iters):
            G.glu_fwd(x, w)
    elif a.op == "glu_bwd":
        dy = torch.randn(a.m, a.k, device=dev).bfloat16()
        wd = (torch.randn(a.k, a.n, device=dev) * 0.02).bfloat16()
        gu = torch.randn(a.m, 2 * a.n, device=dev).bfloat16()
        for _ in range(a.iters):
            G.glu_bwd(dy, wd, gu)
    elif a.op == "rmsnorm":
        from mesh_b200.ops.norm import rmsnorm_fwd
        x = torch.randn(a.m * 8, a.n, device=dev).bfloat16()
        w = torch.ones(a.n, device=dev).bfloat16()
        for _ in range(a.iters):
            rmsnorm_fwd(x, w)
    elif a.op == "rope":
        from mesh_b200.ops.rope import rope_, rope_tables
        cos, sin = rope_tables(4096, 256, 1e6)
        x = torch.randn(a.m * 8, 8, 256, device=dev).bfloat16()
        pos = torch.randint(0, 4096, (a.m * 8,), device=dev, dtype=torch.int32)
        for _ in range(a.iters):
            rope_(x, pos, cos, sin)
    elif a.op == "router":
        from mesh_b200.ops.router import router_topk
        logits = torch.randn(a.m * 64, 64, device=dev)
        for _ in range(a.iters):
            router_topk(logits, 6)
    elif a.op in ("flash_fwd", "flash_bwd"):
        from mesh_b200.ops.attention import flash_attention, flash_attention_backward
        T, H, hd = a.m, a.n if a.n <= 64 else 8, a.k if a.k <= 256 else 128
        B = 4
        q, k, v = (torch.randn(B, T, H, hd, device=dev).bfloat16() for _ in range(3))
        out, lse = flash_attention(q, k, v, causal=True, need_lse=True)
        dout = torch.randn_like(out)
        delta = (dout.float() * out.float()).sum(-1).transpose(1, 2).contiguous()
        if a.op == "flash_fwd":
            run = lambda: flash_attention(q, k, v, causal=True, need_lse=True)
            flops = 4 * B * H * T * T * hd / 2
        else:
            dq = torch.zeros(B, T, H, hd, device=dev)
            run = lambda: flash_attention_backward(q, k, v, out, lse, dout, causal=True, delta=delta, dq=dq)
            flops = 10 * B * H * T * T * hd / 2
        for _ in range(a.iters):
            run()
        if a.time:
            _time(run, flops, f"{a.op} B{B} T{T} H{H} hd{hd} causal")
    elif a.op == "decode_linear":
        from mesh_b200.ops import decode as D
        # several weight matrices in turn, so that the weights come from HBM and not from L2
        n_w = max(2, (256 << 20) // (a.n * a.k * 2))
        ws = [(torch.randn(a.n, a.k, device=dev) * 0.02).bfloat16() for _ in range(n_w)]
        B = a.m if a.m <= 8 else 1
        x = torch.randn(B, a.k, device=dev).bfloat16()
        out = torch.empty(B, a.n, device=dev, dtype=torch.bfloat16)
        state = {"i": 0}

        def run():
            D.decode_linear(x, ws[state["i"] % n_w], out=out)
            state["i"] += 1
        for _ in range(a.iters):
            run()
        if a.time:
            _time(run, 0, f"decode_linear B{B} {a.n}x{a.k} bf16", bytes_moved=a.n * a.k * 2)
    elif a.op == "e2b_decode":
        # solo E2B-class decoder: short prefill, then `iters` eager decode steps (152 launches each)
        import torch.distributed as dist
        from mesh_b200.distributed.context import MeshContext
        from mesh_b200.models.e2b import E2BConfig, E2BDecoder
        from mesh_b200.runtime.rendezvous import Rendezvous
        ctx = MeshContext(0, 1, torch.device("cuda", 0), Rendezvous(dist.HashStore(), 0, 1), None)
        m = E2BDecoder(E2BConfig(), ctx, a.m if a.m <= 8 else 1, "w4" if a.n == 4 else "bf16")
        prompt = torch.randint(0, 262144, (m.B, 64), dtype=torch.int32, device=dev)
        m.prefill(prompt)
        if a.k != 4096:
            m.pos.fill_(a.k)                              # --k <position>: how many keys the attention sees
        torch.cuda.synchronize()
        for _ in range(a.iters):
            m._decode_step()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()                       # with `ncu --profile-from-start off`: only this step is listed
        m._decode_step()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    elif a.op == "e2b_step_timeline":
        # the decode step as one cooperative kernel: per kind of operation, microseconds on the first CTA (device clock)
        import collections
        import json
        import torch.distributed as dist
        from mesh_b200.distributed.context import MeshContext
        from mesh_b200.models.e2b import E2BConfig, E2BDecoder
        from mesh_b200.runtime.rendezvous import Rendezvous
        ctx = MeshContext(0, 1, torch.device("cuda", 0), Rendezvous(dist.HashStore(), 0, 1), None)
        m = E2BDecoder(E2BConfig(), ctx, a.m if a.m <= 8 else 1, {4: "w4", 8: "w8"}.get(a.n, "bf16"))
        prompt = torch.randint(0, 262144, (m.B, 512), dtype=torch.int32, device=dev)
        m.prefill(prompt)
        m.capture("step")
        m.decode(5, record=False)
        torch.cuda.synchronize()
        tl = m.stepk.timeline()
        agg: dict = collections.OrderedDict()
        prev_end = 0.0
        for r in tl:
            d = agg.setdefault(r["op"], {"n": 0, "body_us": 0.0, "waited_us": 0.0, "gap_us": 0.0})
            d["n"] += 1
            d["body_us"] += r["end_us"] - r["start_us"]
            d["waited_us"] += r["waited_us"]
            d["gap_us"] += r["start_us"] - prev_end
            prev_end = r["end_us"]
        print(json.dumps({"weights": m.quant, "batch": m.B, "grid": m.stepk.grid, "smem": m.stepk.smem,
                          "step_us": round(tl[-1]["end_us"], 1),
                          "per_kind": {k: {x: round(y, 1) for x, y in v.items()} for k, v in agg.items()}}))
    else:
        raise SystemExit(f"unknown op {a.op}")
    check_status()
    torch.cuda.synchronize()
    print("ok")


if __name__ == "__main__":
    main()
