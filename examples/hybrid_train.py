#!/usr/bin/env python3
"""Training a decoder under tensor x context x pipeline x data parallelism at once, eagerly, on this package's
kernels: fused all-gather->GEMM / GEMM->reduce-scatter FFN over the tensor axis, ring attention over the context axis,
one-forward-one-backward over the pipeline axis (NCCL point-to-point), sharded AdamW over the data axis.

    python -m torch.distributed.run --nproc-per-node 8 examples/hybrid_train.py --grid tp2cp2pp2 --steps 5

Without a launcher it runs the same model on one device (CPU in fp32 if there is no GPU)."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--grid", default="solo")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--micro", type=int, default=2)
    ap.add_argument("--small", action="store_true")
    a = ap.parse_args(argv)
    from mesh_b200.models.hybrid import HybridConfig, HybridTrainer
    from mesh_b200.parallel.topology import ParallelContext, ParallelDims
    dims = ParallelDims.parse(a.grid)
    cuda = torch.cuda.is_available()
    ctx = None
    if dims.world > 1 or "RANK" in os.environ:
        from mesh_b200.distributed import init
        ctx = init(backend="nccl" if cuda else "gloo")
    par = ParallelContext(ctx, dims)
    if not cuda:
        par.device = torch.device("cpu")
    cfg = HybridConfig(vocab=256, d_model=64, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128, seq_len=32) if (a.small or not cuda) \
        else HybridConfig(vocab=8192, d_model=1024, n_layers=8, n_heads=8, n_kv_heads=8, head_dim=128, d_ff=4096, seq_len=2048)
    tr = HybridTrainer(cfg, par, micro_batch=1, n_micro=a.micro, lr=3e-3, dtype=torch.bfloat16 if cuda else torch.float32)
    g = torch.Generator().manual_seed(1 + par.dp.rank)
    tokens = torch.randint(0, cfg.vocab, (a.micro, cfg.seq_len), generator=g).to(par.device)
    losses = [float(tr.step(tokens, tokens.roll(-1, 1))) for _ in range(a.steps)]
    if par.rank == 0:
        print(json.dumps({"grid": str(dims), "losses": [round(l, 4) for l in losses], "decreasing": losses[-1] < losses[0],
                          "pipeline": tr.stats}), flush=True)
    if ctx is not None:
        from mesh_b200.distributed import shutdown
        shutdown()
    return losses


if __name__ == "__main__":
    main()
