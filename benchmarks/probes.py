"""Machine probes: HBM copy bandwidth, dense bf16 GEMM rate (this package's tcgen05 kernel and cuBLAS), and, with
more than one rank, peer-to-peer bandwidth / latency and collective bus bandwidth for this package's kernels and for
NCCL.  The figures are the denominators of the roofline reports (the reference keeps such probes under ``bench/``
and ``user/bench``: link bandwidth, latency, memory copy)."""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from common import emit, init, time_steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    a = ap.parse_args()
    ctx = init()
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    from mesh_b200.ops.gemm import gemm
    from mesh_b200.ops.norm import rmsnorm_fwd
    from mesh_b200.utils.status import check_status
    rec = {"metric": "machine_probes", "n_gpus": world}
    # ---- memory
    n = 1 << 30
    src, dst = torch.empty(n, dtype=torch.uint8, device=dev), torch.empty(n, dtype=torch.uint8, device=dev)
    ms = time_steps(lambda: dst.copy_(src), a.steps, 3, world, dev, flush_l2=False)
    rec["hbm_copy_gbs"] = round(2 * n / ms / 1e6, 1)
    x = torch.randn(65536, 4096, device=dev).bfloat16()
    w = torch.ones(4096, device=dev, dtype=torch.bfloat16)
    ms = time_steps(lambda: rmsnorm_fwd(x, w), a.steps, 3, world, dev, flush_l2=False)
    rec["rmsnorm_kernel_gbs"] = round(2 * x.numel() * 2 / ms / 1e6, 1)
    del src, dst, x
    # ---- tensor cores
    A = torch.randn(8192, 8192, device=dev).bfloat16()
    B = torch.randn(8192, 8192, device=dev).bfloat16()
    fl = 2 * 8192 ** 3
    ms = time_steps(lambda: gemm(A, B), a.steps, 3, world, dev, flush_l2=False)
    rec["gemm_tcgen05_tflops"] = round(fl / ms / 1e9, 1)
    ms = time_steps(lambda: torch.matmul(A, B.T), a.steps, 3, world, dev, flush_l2=False)
    rec["gemm_cublas_tflops"] = round(fl / ms / 1e9, 1)
    del A, B
    # ---- links
    if world > 1:
        comm = ctx.comm
        big = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        out = torch.empty_like(big)
        ring = [(j, (j + 1) % world) for j in range(world)]
        ms = time_steps(lambda: comm.permute(out, big, ring), a.steps, 3, world, dev, flush_l2=False)
        rec["p2p_ring_gbs_per_direction"] = round(big.numel() / ms / 1e6, 1)
        ms = time_steps(lambda: dist.batch_isend_irecv([dist.P2POp(dist.isend, big, (rank + 1) % world),
                                                        dist.P2POp(dist.irecv, out, (rank - 1) % world)])[-1].wait(),
                        a.steps, 3, world, dev, flush_l2=False)
        rec["p2p_ring_nccl_gbs_per_direction"] = round(big.numel() / ms / 1e6, 1)
        mid = torch.empty(8 << 20, dtype=torch.uint8, device=dev)
        omid = torch.empty_like(mid)
        ms = time_steps(lambda: comm.permute(omid, mid, ring), a.steps, 3, world, dev, flush_l2=False, inner=10)
        rec["p2p_ring_8MiB_us"] = round(ms * 1e3, 1)
        small = torch.zeros(16, dtype=torch.uint8, device=dev)
        outs = torch.zeros_like(small)
        pairs = [(0, 1), (1, 0)]
        ms = time_steps(lambda: comm.permute(outs, small, pairs), 10, 5, world, dev, flush_l2=False, inner=50)
        rec["p2p_exchange_16B_us"] = round(ms * 1e3, 2)
        sizes = [8 << 10, 256 << 10, 8 << 20, 256 << 20]
        rows = []
        for nb in sizes:
            t = torch.ones(nb // 2, dtype=torch.bfloat16, device=dev)
            inner = 50 if nb <= (1 << 20) else 4
            t_mesh = time_steps(lambda: comm.all_reduce(t), a.steps, 3, world, dev, flush_l2=False, inner=inner)
            t_nccl = time_steps(lambda: dist.all_reduce(t), a.steps, 3, world, dev, flush_l2=False, inner=inner)
            bus = 2 * (world - 1) / world * nb
            rows.append({"bytes": nb, "mesh_us": round(t_mesh * 1e3, 1), "nccl_us": round(t_nccl * 1e3, 1),
                         "mesh_busbw_gbs": round(bus / t_mesh / 1e6, 1), "nccl_busbw_gbs": round(bus / t_nccl / 1e6, 1)})
        rec["all_reduce"] = rows
        rows = []
        for nb in (1 << 20, 64 << 20):
            part = torch.ones(nb // 2 // world, dtype=torch.bfloat16, device=dev)
            full = torch.empty(nb // 2, dtype=torch.bfloat16, device=dev)
            kw = dict(flush_l2=False, inner=20 if nb <= (1 << 20) else 4)
            t_ag = time_steps(lambda: comm.all_gather(full, part), a.steps, 3, world, dev, **kw)
            t_ag_n = time_steps(lambda: dist.all_gather_into_tensor(full, part), a.steps, 3, world, dev, **kw)
            t_rs = time_steps(lambda: comm.reduce_scatter(part, full), a.steps, 3, world, dev, **kw)
            t_rs_n = time_steps(lambda: dist.reduce_scatter_tensor(part, full), a.steps, 3, world, dev, **kw)
            rows.append({"bytes": nb, "all_gather_mesh_us": round(t_ag * 1e3, 1), "all_gather_nccl_us": round(t_ag_n * 1e3, 1),
                         "reduce_scatter_mesh_us": round(t_rs * 1e3, 1), "reduce_scatter_nccl_us": round(t_rs_n * 1e3, 1)})
        rec["gather_scatter"] = rows
    check_status()
    emit(rank, rec)
    from mesh_b200.distributed import shutdown
    shutdown()


if __name__ == "__main__":
    main()
