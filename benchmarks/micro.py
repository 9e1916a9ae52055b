"""Small numerical workloads timed one by one: the shapes the reference's micro-benchmarks probe (bench/peak.py,
prec.py, orth.py, residual.py, pairwise_distance.py, sparse.py, meanfield.py, moe_dispatch.py - there for Apple GPUs
through MLX), stated in PyTorch so that they run on a B200 (or, with ``--device cpu --small``, anywhere).

    python benchmarks/micro.py peak | orth | gram | pairwise | sparse | meanfield | moe_dispatch | all [--small]

Every workload prints one JSON line per variant: milliseconds (CUDA events on a GPU, the host clock on CPU), useful
FLOP/s, and - where variants must agree - the largest difference from the first variant.
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def _timed(fn, device, steps: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / steps
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    return (time.perf_counter() - t0) * 1e3 / steps


def _emit(workload: str, variant: str, ms: float, flops: float, **more) -> dict:
    rec = {"workload": workload, "variant": variant, "ms": round(ms, 4), "gflops": round(flops / (ms * 1e-3) / 1e9, 1), **more}
    print(json.dumps(rec), flush=True)
    return rec


# ----------------------------------------------------------------------------- GEMM rate by dtype
def peak(dev, small: bool, steps: int) -> list:
    n, k = (512, 256) if small else (8192, 8192)
    out = []
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        a, x = torch.randn(n, n, device=dev, dtype=dt), torch.randn(n, k, device=dev, dtype=dt)
        out.append(_emit("peak", str(dt).split(".")[-1], _timed(lambda: a @ x, dev, steps), 2.0 * n * n * k, n=n, k=k))
    if dev.type == "cuda":                                    # this package's tcgen05 kernel on the same product
        import os
        import sys
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        from mesh_b200.ops.gemm import linear
        xt = x.T.contiguous()                                 # linear(a, w) = a w^T
        out.append(_emit("peak", "bfloat16_tcgen05", _timed(lambda: linear(a, xt), dev, steps), 2.0 * n * n * k, n=n, k=k,
                         difference=round(float((linear(a, xt).float() - (a @ x).float()).abs().max() / (a @ x).float().abs().max()), 5)))
    return out


# ----------------------------------------------------------------------------- whitening: X -> X G^{-1/2}-like factors
def _inverse_sqrt_newton_schulz(a: torch.Tensor, iters: int) -> torch.Tensor:
    """``a^{-1/2}`` of a symmetric positive definite matrix by the coupled Newton-Schulz iteration (matrix products
    only): scale to unit diagonal and unit Frobenius norm, iterate ``T = (3I - Z Y) / 2; Y <- Y T; Z <- T Z``."""
    d = torch.rsqrt(a.diagonal())
    s = a * d[:, None] * d[None, :]
    c = s.norm()
    y, eye = s / c, torch.eye(a.shape[0], device=a.device, dtype=a.dtype)
    z = eye.clone()
    for _ in range(iters):
        t = 0.5 * (3.0 * eye - z @ y)
        y, z = y @ t, t @ z
    return d[:, None] * (z * torch.rsqrt(c))


def _blocked_cholesky(a: torch.Tensor, block: int):
    """Recursive Cholesky that returns ``(L, L^{-1})``: the leaves use the library routine, everything above is
    matrix products."""
    r = a.shape[0]
    if r <= block:
        low = torch.linalg.cholesky(a)
        return low, torch.linalg.solve_triangular(low, torch.eye(r, device=a.device, dtype=a.dtype), upper=False)
    h = r // 2
    l11, i11 = _blocked_cholesky(a[:h, :h], block)
    l21 = a[h:, :h] @ i11.T
    l22, i22 = _blocked_cholesky(a[h:, h:] - l21 @ l21.T, block)
    zero = a.new_zeros(h, r - h)
    low = torch.cat([torch.cat([l11, zero], 1), torch.cat([l21, l22], 1)], 0)
    inv = torch.cat([torch.cat([i11, zero], 1), torch.cat([-(i22 @ (l21 @ i11)), i22], 1)], 0)
    return low, inv


def orth(dev, small: bool, steps: int) -> list:
    """Orthonormalise the columns of ``X [n, r]`` against their Gram matrix ``G = X^T X + ridge I``."""
    n, r = (512, 64) if small else (65536, 1024)
    x = torch.randn(n, r, device=dev, dtype=torch.float32)
    gram = lambda: x.T @ x + 1e-3 * torch.eye(r, device=dev)
    flops = 2.0 * n * r * r * 2 + r ** 3 / 3

    def by_cholesky():
        low = torch.linalg.cholesky(gram())
        return torch.linalg.solve_triangular(low, x.T, upper=False).T

    def by_blocked():
        _, inv = _blocked_cholesky(gram(), 16 if small else 256)
        return x @ inv.T

    def by_newton_schulz():
        return x @ _inverse_sqrt_newton_schulz(gram(), 18)

    out = []
    eye = torch.eye(r, device=dev)
    for name, fn in (("cholesky_solve", by_cholesky), ("blocked_cholesky", by_blocked), ("newton_schulz", by_newton_schulz)):
        q = fn()
        err = float((q.T @ q - eye).abs().max())                    # all variants must give orthonormal columns
        out.append(_emit("orth", name, _timed(fn, dev, steps), flops, n=n, r=r, orthogonality_error=round(err, 6)))
    return out


def gram(dev, small: bool, steps: int) -> list:
    n, r = (512, 64) if small else (65536, 512)
    x = torch.randn(n, r, device=dev)

    def step():
        return torch.linalg.cholesky(x.T @ x + 1e-3 * torch.eye(r, device=dev))
    return [_emit("gram", "gram_then_cholesky", _timed(step, dev, steps), 2.0 * n * r * r + r ** 3 / 3, n=n, r=r)]


# ----------------------------------------------------------------------------- pairwise distances through one GEMM
def pairwise(dev, small: bool, steps: int) -> list:
    b, d = (256, 32) if small else (16384, 256)
    x = torch.randn(b, d, device=dev)

    def by_gemm():
        n = (x * x).sum(1)
        return n[:, None] + n[None, :] - 2 * (x @ x.T)

    ref = torch.cdist(x, x).pow(2)
    err = float((by_gemm() - ref).abs().max() / ref.abs().max())
    return [_emit("pairwise", "gemm", _timed(by_gemm, dev, steps), 2.0 * b * b * d, points=b, d=d, difference=round(err, 7)),
            _emit("pairwise", "cdist", _timed(lambda: torch.cdist(x, x).pow(2), dev, steps), 2.0 * b * b * d, points=b, d=d)]


# ----------------------------------------------------------------------------- sparse rows by gathering
def sparse(dev, small: bool, steps: int) -> list:
    n, k = (256, 64) if small else (4096, 1024)
    a, x = torch.randn(n, n, device=dev), torch.randn(n, k, device=dev)
    dense_ms = _timed(lambda: a @ x, dev, steps)
    out = [_emit("sparse", "dense", dense_ms, 2.0 * n * n * k, density=1.0)]
    for density in (0.30, 0.10, 0.03, 0.01):
        nnz = max(1, int(n * density))
        idx = torch.randint(0, n, (n, nnz), device=dev)
        val = torch.randn(n, nnz, device=dev)

        def spmm():
            return torch.einsum("rjk,rj->rk", x[idx], val)              # gather the rows each output row needs
        ms = _timed(spmm, dev, steps)
        out.append(_emit("sparse", "gather", ms, 2.0 * n * nnz * k, density=density, nnz_per_row=nnz,
                         speedup_over_dense=round(dense_ms / ms, 3)))
    return out


# ----------------------------------------------------------------------------- a fixed-point solve with exchanges
def meanfield(dev, small: bool, steps: int) -> list:
    """``iterations`` rounds of ``V <- gamma A softplus(R + V - mu rho)``; every fourth round the column sums are
    exchanged (summed over the ranks of the job when there is one: the per-round wire cost is one vector)."""
    import torch.distributed as dist
    n, k = (128, 64) if small else (4096, 1536)
    iterations, gamma, mu = 32, 0.92, 0.35
    a = torch.randn(n, n, device=dev).square()
    a = a / a.sum(1, keepdim=True)
    r = torch.randn(n, k, device=dev)
    shared = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1

    def solve():
        v, rho, exchanges = torch.zeros(n, k, device=dev), torch.zeros(n, device=dev), 0
        for m in range(iterations):
            z = torch.nn.functional.softplus(r + v - mu * rho[:, None])
            v = gamma * (a @ z)
            if m % 4 == 3:
                rho = z.sum(1)
                if shared:
                    dist.all_reduce(rho)
                exchanges += 1
        return v, exchanges

    _, exchanges = solve()
    ms = _timed(lambda: solve(), dev, max(1, steps // 2), warmup=1)
    return [_emit("meanfield", "solve", ms, iterations * k * (2.0 * n * n + 8 * n), n=n, k=k, exchanges=exchanges,
                  bytes_per_exchange=n * 4, solves_per_second=round(1e3 / ms, 2))]


# ----------------------------------------------------------------------------- expert dispatch by index
def moe_dispatch(dev, small: bool, steps: int) -> list:
    """Top-1 routed expert FFN, three ways: gather every token's expert matrices (``unsorted``), sort the tokens by
    expert and run one product per expert (``sorted``), pad every expert to the same number of rows and use one
    batched product (``padded``)."""
    t, d, f, e = (256, 32, 64, 4) if small else (16384, 1024, 2048, 16)
    dt = torch.float32 if dev.type == "cpu" else torch.bfloat16
    x = torch.randn(t, d, device=dev, dtype=dt)
    w1 = torch.randn(e, d, f, device=dev, dtype=dt) * d ** -0.5
    w2 = torch.randn(e, f, d, device=dev, dtype=dt) * f ** -0.5
    expert = torch.randint(0, e, (t,), device=dev)
    flops = 4.0 * t * d * f

    def unsorted():
        h = torch.relu(torch.bmm(x[:, None, :], w1[expert]))           # [t, 1, f]: reads one matrix pair per token
        return torch.bmm(h, w2[expert])[:, 0]

    def by_sorting():
        order = torch.argsort(expert)
        counts = torch.bincount(expert, minlength=e).tolist()
        xs, out, at = x[order], torch.empty_like(x), 0
        for j, c in enumerate(counts):
            if c:
                out[at:at + c] = torch.relu(xs[at:at + c] @ w1[j]) @ w2[j]
                at += c
        back = torch.empty_like(out)
        back[order] = out
        return back

    def padded():
        order = torch.argsort(expert)
        counts = torch.bincount(expert, minlength=e)
        cap = int(counts.max())
        start = torch.cumsum(counts, 0) - counts
        slot = torch.arange(t, device=dev) - start[expert[order]]       # position of each sorted token within its expert
        buf = x.new_zeros(e, cap, d)
        buf[expert[order], slot] = x[order]
        y = torch.bmm(torch.relu(torch.bmm(buf, w1)), w2)
        back = torch.empty_like(x)
        back[order] = y[expert[order], slot]
        return back

    out, ref = [], None
    small_steps = max(1, steps // 4) if not small else steps
    for name, fn, n_steps in (("sorted", by_sorting, steps), ("padded", padded, steps), ("unsorted", unsorted, small_steps)):
        if name == "unsorted" and not small and t * d * f * x.element_size() > (8 << 30):
            continue                                                    # the gathered matrices would not fit
        y = fn().float()
        ref = y if ref is None else ref
        err = float((y - ref).abs().max() / ref.abs().max())
        out.append(_emit("moe_dispatch", name, _timed(fn, dev, n_steps), flops, tokens=t, d=d, f=f, experts=e, difference=round(err, 5)))
    return out


WORKLOADS = {"peak": peak, "orth": orth, "gram": gram, "pairwise": pairwise, "sparse": sparse, "meanfield": meanfield,
             "moe_dispatch": moe_dispatch}


def main(argv=None) -> list:
    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=[*WORKLOADS, "all"])
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    torch.manual_seed(0)
    names = list(WORKLOADS) if a.workload == "all" else [a.workload]
    out = []
    for n in names:
        out += WORKLOADS[n](dev, a.small, a.steps)
    return out


if __name__ == "__main__":
    main()
