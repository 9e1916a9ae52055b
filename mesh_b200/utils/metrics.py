"""Observability: JSON-lines step log, workload envelopes, roofline fractions, and an opt-in ledger.

* ``StepLog``: one JSON line per step and rank (the reference's example reports are single-line JSON,
  examples/parallel.py:217).
* ``WorkloadMeter`` / ``span``: FLOP and byte envelopes per stage, from which the achieved fraction of the
  machine's capacity is estimated (rdma/workload.py:84-134, viz/serve.py:280-338).
* ``roofline``: the report every fused kernel is judged by — the slower of compute at the measured peak and
  bytes over NVLink (or HBM) at the measured bandwidth.
* ``Ledger``: MESH_LEDGER-style opt-in trace of (name, start, end) device times per collective / kernel
  (rdma/mesh-flow.c:1047-1064); off by default so the normal path pays nothing.
"""
from __future__ import annotations

import contextlib
import json
import os
import time

import torch

from ..config import capacity, config


class StepLog:
    def __init__(self, path: str | None = None, rank: int = 0):
        self.path = path or config().metrics_path
        self.rank = rank
        self._f = open(self.path, "a") if self.path else None

    def write(self, **fields) -> None:
        if self._f is None:
            return
        fields.setdefault("t", time.time())
        fields.setdefault("rank", self.rank)
        self._f.write(json.dumps(fields, sort_keys=True) + "\n")
        self._f.flush()

    def close(self) -> None:
        if self._f:
            self._f.close()
            self._f = None


def roofline(flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0, seconds: float | None = None,
             sustained: bool = False) -> dict:
    """Target time = max(FLOPs / measured GEMM peak, HBM bytes / measured copy bandwidth, NVLink bytes / measured
    per-direction bandwidth); with ``seconds`` also the achieved fraction of that roofline."""
    cap = capacity()
    peak = cap["bf16_tflops_sustained" if sustained else "bf16_tflops"] * 1e12
    t_c = flops / peak if flops else 0.0
    t_m = hbm_bytes / (cap["hbm_gbs"] * 1e9) if hbm_bytes else 0.0
    t_n = nvlink_bytes / (cap["nvlink_gbs_per_dir"] * 1e9) if nvlink_bytes else 0.0
    target = max(t_c, t_m, t_n)
    out = {"compute_s": t_c, "hbm_s": t_m, "nvlink_s": t_n, "target_s": target,
           "bound": "compute" if target == t_c else ("hbm" if target == t_m else "nvlink")}
    if seconds:
        out["achieved_s"] = seconds
        out["fraction_of_measured_roofline"] = target / seconds if seconds > 0 else None
    return out


class WorkloadMeter:
    """Accumulates FLOP / byte envelopes per named span and reports fractions of capacity."""

    def __init__(self):
        self.spans: list[dict] = []

    @contextlib.contextmanager
    def span(self, name: str, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0):
        cuda = torch.cuda.is_available()
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        yield
        if cuda:
            e1.record()
            e1.synchronize()
            dt = e0.elapsed_time(e1) * 1e-3
        else:
            dt = time.perf_counter() - t0
        rec = {"name": name, "seconds": dt, "flops": flops, "hbm_bytes": hbm_bytes, "nvlink_bytes": nvlink_bytes}
        rec.update(roofline(flops, hbm_bytes, nvlink_bytes, dt))
        self.spans.append(rec)

    def report(self) -> list[dict]:
        return list(self.spans)


class Ledger:
    """Opt-in (``MESH_LEDGER=1``) per-operation device timestamps."""

    def __init__(self, enabled: bool | None = None):
        self.enabled = config().ledger if enabled is None else enabled
        self.records: list = []

    @contextlib.contextmanager
    def record(self, name: str):
        if not self.enabled or not torch.cuda.is_available():
            yield
            return
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        yield
        e1.record()
        self.records.append((name, e0, e1))

    def dump(self) -> list[dict]:
        torch.cuda.synchronize()
        if not self.records:
            return []
        base = self.records[0][1]
        return [{"name": n, "start_us": base.elapsed_time(a) * 1e3, "us": a.elapsed_time(b) * 1e3} for n, a, b in self.records]
