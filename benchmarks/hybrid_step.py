"""Hybrid training step: tensor x context x pipeline (x data) parallel decoder, ring attention over the context
axis, one-forward-one-backward over the microbatches, sharded AdamW; bf16, synthetic token ids, random-init weights.

Default is the full configuration (24 layers, d_model 2048, 16 heads of 128, FFN 8192, vocab 50304, sequence 8192,
8 microbatches of one sequence, grid tp2 x cp2 x pp2 on 8 GPUs); ``--small`` shrinks it for a quick check.
"""
from __future__ import annotations

import argparse

import torch

from common import barrier, emit, init


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--grid", default="tp2cp2pp2")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--micro", type=int, default=8)
    ap.add_argument("--impl", choices=["mesh", "stock"], default="mesh",
                    help="stock: the same model and grid from PyTorch's own modules and torch.distributed (baseline/hybrid_stock.py)")
    a = ap.parse_args()
    if a.impl == "stock":
        return stock(a)
    from mesh_b200.config import MeshConfig, set_config
    set_config(MeshConfig.from_env(heap_bytes=16 << 30))      # gathered activations of every layer live in the heap
    ctx = init()
    from mesh_b200 import _native
    from mesh_b200.models.hybrid import HybridConfig, HybridTrainer
    from mesh_b200.parallel.topology import ParallelContext, ParallelDims
    from mesh_b200.utils.status import check_status
    dims = ParallelDims.parse(a.grid)
    par = ParallelContext(ctx, dims)
    if a.small:
        cfg = HybridConfig(vocab=8192, d_model=1024, n_layers=4, n_heads=8, n_kv_heads=8, head_dim=128, d_ff=4096, seq_len=2048)
    else:
        cfg = HybridConfig(vocab=50304, d_model=2048, n_layers=24, n_heads=16, n_kv_heads=16, head_dim=128, d_ff=8192,
                           seq_len=8192)
    M = a.micro
    tr = HybridTrainer(cfg, par, micro_batch=1, n_micro=M, lr=1e-4)
    g = torch.Generator(device="cpu").manual_seed(3 + par.dp.rank)
    tokens = torch.randint(0, cfg.vocab, (M, cfg.seq_len), generator=g).pin_memory()
    targets = torch.randint(0, cfg.vocab, (M, cfg.seq_len), generator=g).pin_memory()
    dev = ctx.device

    def step():
        return tr.step(tokens.to(dev, non_blocking=True), targets.to(dev, non_blocking=True))

    for _ in range(max(1, a.warmup)):
        loss = step()
    barrier(ctx.world)
    l0 = _native.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    last = float(loss)                                    # device -> host read of the step's result
    barrier(ctx.world)
    ms = e0.elapsed_time(e1) / a.steps
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if ctx.world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms = float(t[0])
    check_status()
    tok = M * cfg.seq_len * dims.dp
    n_params = cfg.n_layers * (cfg.d_model * (cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim + cfg.n_heads * cfg.head_dim * cfg.d_model
                               + 3 * cfg.d_model * cfg.d_ff) + 2 * cfg.vocab * cfg.d_model
    flops = 6 * n_params * tok + 6 * cfg.n_layers * tok * cfg.seq_len * cfg.n_heads * cfg.head_dim   # causal attention: half of 12
    emit(ctx.rank, {"metric": "hybrid_train_tokens_per_s", "value": round(tok / (ms * 1e-3), 1), "unit": "tokens/s",
                    "n_gpus": ctx.world, "ms_per_step": round(ms, 3), "steps": a.steps, "loss": round(last, 4),
                    "model_tflops_per_gpu": round(flops / (ms * 1e-3) / 1e12 / ctx.world, 1),
                    "gpu_launches_per_step": (_native.launch_count - l0) // a.steps,
                    "pipeline": tr.stats,
                    "config": {"grid": str(dims), "layers": cfg.n_layers, "d_model": cfg.d_model, "heads": cfg.n_heads,
                               "d_ff": cfg.d_ff, "vocab": cfg.vocab, "seq_len": cfg.seq_len, "microbatches": M,
                               "attention": "ring over cp, striped tokens", "optimizer": "AdamW bf16 params, fp32 state",
                               "inputs": "pinned host token ids copied every step"}})
    from mesh_b200.distributed import shutdown
    shutdown()


def stock(a):
    """The stock arm: same configuration, same clock, none of this package's kernels, layers or collectives."""
    import os

    import torch.distributed as dist
    sys_path_root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    import sys
    sys.path.insert(0, sys_path_root)
    from baseline.hybrid_stock import Grid, StockConfig, StockTrainer
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    grid = Grid(a.grid if world > 1 else "", rank, world)
    if a.small:
        cfg = StockConfig(vocab=8192, d_model=1024, n_layers=4, n_heads=8, n_kv_heads=8, head_dim=128, d_ff=4096, seq_len=2048)
    else:
        cfg = StockConfig(vocab=50304, d_model=2048, n_layers=24, n_heads=16, n_kv_heads=16, head_dim=128, d_ff=8192, seq_len=8192)
    M = a.micro
    tr = StockTrainer(cfg, grid, dev, torch.bfloat16, micro_batch=1, n_micro=M, lr=1e-4)
    g = torch.Generator(device="cpu").manual_seed(3 + grid.coord["dp"])
    tokens = torch.randint(0, cfg.vocab, (M, cfg.seq_len), generator=g).pin_memory()
    targets = torch.randint(0, cfg.vocab, (M, cfg.seq_len), generator=g).pin_memory()

    def step():
        return tr.step(tokens.to(dev, non_blocking=True), targets.to(dev, non_blocking=True))

    for _ in range(max(1, a.warmup)):
        loss = step()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    last = float(loss)
    barrier(world)
    t = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    tok = M * cfg.seq_len * grid.size["dp"]
    emit(rank, {"metric": "hybrid_train_tokens_per_s", "impl": "stock", "value": round(tok / (ms * 1e-3), 1), "unit": "tokens/s",
                "n_gpus": world, "ms_per_step": round(ms, 3), "steps": a.steps, "loss": round(last, 4),
                "config": {"grid": a.grid if world > 1 else "solo", "layers": cfg.n_layers, "d_model": cfg.d_model,
                           "heads": cfg.n_heads, "d_ff": cfg.d_ff, "vocab": cfg.vocab, "seq_len": cfg.seq_len, "microbatches": M,
                           "attention": "scaled_dot_product_attention; keys and values all-gathered over cp, contiguous tokens",
                           "pipeline": "all forward, then all backward", "optimizer": "torch.optim.AdamW fused, bf16 parameters",
                           "inputs": "pinned host token ids copied every step"}})
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
