"""Shared command line and report of the example programs.

Every example builds a model, states a placement, compiles it for a set of processors, runs the compiled program and
compares it with eager PyTorch, then prints one JSON line: channels by kind, the schedule signature, the error against
eager (the reference's examples report the same things, examples/parallel.py:190-218).

By default the processors are CPU threads of this process, so an example runs anywhere; under ``torchrun`` (one process
per GPU) the same program runs with one processor per rank on CUDA.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def arguments(description: str, argv=None):
    ap = argparse.ArgumentParser(description=description)
    ap.add_argument("--nodes", type=int, default=2, help="processors (ignored under torchrun: one per rank)")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--units", default=None, help="share ratios 'a,b,...' or 'striped'")
    ap.add_argument("--archive", action="store_true", help="save the compiled program, load it back, run the copy")
    ap.add_argument("--times", type=int, default=1, help="timed executions")
    ap.add_argument("--small", action="store_true", help="shrink the model (tests)")
    return ap.parse_args(argv)


def units_of(args):
    if args.units in (None, "", "none"):
        return None
    if args.units == "striped":
        return "striped"
    return tuple(float(u) for u in args.units.split(","))


def processors(args) -> dict:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        return {f"rank{r}": (0, f"cuda:{r}" if args.device.startswith("cuda") else "cpu") for r in range(world)}
    return {f"p{i}": (0, args.device) for i in range(args.nodes)}


def execute(model, inputs, placement, args, *, loss=None, functions=None, mesh=None, tol=2e-4) -> dict:
    """compile -> (archive round trip) -> run -> compare with eager -> one-line JSON report."""
    from mesh_b200.compiler import Program, compile_module, compile_program
    from mesh_b200.compiler import archive
    procs = processors(args)
    t0 = time.perf_counter()
    kw = {} if loss is None else {"loss": loss}
    if functions:
        sch = compile_program(model, inputs, functions, procs, placement(tuple(procs)), mesh=mesh, **kw)
    else:
        sch = compile_module(model, inputs, procs, placement(tuple(procs)), mesh=mesh, **kw)
    t_compile = time.perf_counter() - t0
    if args.archive:
        with tempfile.TemporaryDirectory() as d:
            archive.save(d, sch)
            sch = archive.load(d)
    prog = Program(sch)
    res = prog(*inputs)
    t0 = time.perf_counter()
    for _ in range(args.times):
        res = prog(*inputs)
    t_run = (time.perf_counter() - t0) / max(1, args.times)
    # eager reference
    if loss is not None:
        for p in model.parameters():
            p.grad = None
        ref = model(*inputs)
        ref_loss = ref if torch.is_tensor(ref) else ref[loss]
        ref_loss.backward()
        got = res.outputs if torch.is_tensor(res.outputs) else res.outputs[loss]
        err = abs(float(got.detach()) - float(ref_loss.detach()))
        err /= max(1.0, abs(float(ref_loss)))
        names = dict(model.named_parameters())
        for k, g in res.parameters.items():
            want = names[k].grad
            if g.shape == want.shape:
                err = max(err, float((g - want).abs().max() / (want.abs().max() + 1e-9)))
    else:
        with torch.no_grad():
            ref = model(*inputs)
        flat_res = res if isinstance(res, (tuple, list)) else (res,)
        flat_ref = ref if isinstance(ref, (tuple, list)) else (ref,)
        err = max(float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)) for a, b in zip(flat_res, flat_ref))
    s = sch.structure
    report = {"processors": len(procs), "channels": s.get("channels"), "by_kind": s.get("by_kind"), "by_verb": s.get("by_verb"),
              "signature": getattr(sch.signature, "digest", None) or str(sch.signature)[:40], "signature_ok": sch.signature.ok(),
              "error": err, "ok": bool(err < tol), "compile_s": round(t_compile, 3), "run_s": round(t_run, 4)}
    from mesh_b200.compiler.devices import crossings
    cross = crossings(sch.plan, procs)
    report["bytes_between_processors"] = s.get("bytes_between_processors")
    report["between_machines"] = {"transfers": cross["between_machines"], "bytes": cross["bytes_between_machines"]}
    if "function_calls" in s:
        report["function_calls"] = s["function_calls"]
    print(json.dumps(report, default=str), flush=True)
    return report
