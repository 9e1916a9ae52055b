#!/usr/bin/env python3
"""Greedy decoding with an E2B-class decoder (sliding-window / global attention 4:1, GeGLU, tied vocabulary of 262144)
on the decode kernels: one CUDA graph per token, tensor parallel over all ranks when run under a launcher.

    python examples/decode_e2b.py --batch 8 --weights w4
    python -m torch.distributed.run --nproc-per-node 4 examples/decode_e2b.py
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--weights", default="bf16", choices=["bf16", "w4"])
    ap.add_argument("--prompt", type=int, default=128)
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--layers", type=int, default=30)
    a = ap.parse_args(argv)
    from mesh_b200.distributed import init, shutdown
    from mesh_b200.models.e2b import E2BConfig, E2BDecoder
    ctx = init(backend="nccl")
    cfg = E2BConfig(layers=a.layers)
    m = E2BDecoder(cfg, ctx, a.batch, a.weights)
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, cfg.vocab, (a.batch, a.prompt), generator=g, dtype=torch.int32).to(ctx.device)
    m.prefill(prompt)
    m.capture()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    out = m.decode(a.tokens)
    e1.record()
    torch.cuda.synchronize()
    if ctx.rank == 0:
        ms = e0.elapsed_time(e1)
        print(json.dumps({"tp": ctx.world, "batch": a.batch, "weights": a.weights, "tokens_per_s": round(a.batch * a.tokens / ms * 1e3, 1),
                          "first_tokens": out[:8, 0].tolist()}), flush=True)
    shutdown()


if __name__ == "__main__":
    main()
