#!/usr/bin/env python3
"""A hybrid job as ONE compiled program: pipeline stages x context parallelism x tensor parallelism on a grid of
processors (``--grid pp,cp,tp``, default 2,2,2), forward and backward.

The decoder's layers are split over the pipeline axis by their module paths, the tokens over the context axis, the
projections Megatron-fashion over the tensor axis (``mesh_b200.compiler.placements.grid``); the compiler derives every
transfer: point-to-point crossings between the stages, gathers of keys and values along the context axis (one ring
step per attention in inference graphs), all-reduces of the row-parallel partial sums and of the gradients.  The eager
counterpart with hand-written schedules is ``examples/hybrid_train.py``.

    python examples/hybrid_compiled.py --small                  # 8 CPU threads
    python examples/hybrid_compiled.py --small --grid 2,1,2 --inference
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--grid", default="2,2,2", help="processors along the pipeline, context and tensor axes")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--inference", action="store_true", help="forward only (attention stays one operator: ring steps)")
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    from mesh_b200.compiler import Program, compile_module, placements
    from mesh_b200.models.llama import Decoder
    pp, cp, tp = (int(v) for v in a.grid.split(","))
    dim, heads, ffn, layers, batch, seq = (32, 4, 64, 2 * pp, 2, 8 * cp) if a.small else (1024, 16, 4096, 4 * pp, 2, 512 * cp)
    torch.manual_seed(0)
    model = Decoder(dim=dim, heads=heads, ffn=ffn, layers=layers)
    x = torch.randn(batch, seq, dim)
    per = layers // pp
    stages = {"|".join(rf"blocks\.{i}\." for i in range(k * per, (k + 1) * per)): k for k in range(pp)}
    place = placements.grid(("pp", "cp", "tp"), stages=stages, stage_axis="pp", column=("wq", "wk", "wv", "w1", "w3"),
                            row=("wo", "w2"), tensor_axis="tp", inputs={"x": {"cp": 1}})
    procs = {f"s{r // (cp * tp)}c{(r // tp) % cp}t{r % tp}": (0, a.device) for r in range(pp * cp * tp)}
    if a.inference:
        blocks = model.blocks

        class Body(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.blocks = blocks

            def forward(self, x):
                for b in self.blocks:
                    x = b(x)
                return x
        model = Body().eval()
    t0 = time.perf_counter()
    sch = compile_module(model, (x,), procs, place, mesh=(pp, cp, tp), **({} if a.inference else {"loss": 0}))
    t_compile = time.perf_counter() - t0
    prog = Program(sch)
    t0 = time.perf_counter()
    res = prog(x)
    t_run = time.perf_counter() - t0
    if a.inference:
        with torch.no_grad():
            ref = model(x)
        err = float((res - ref).abs().max() / ref.abs().max())
    else:
        ref = model(x)
        ref.backward()
        err = abs(float(res.outputs.detach()) - float(ref.detach())) / max(1.0, abs(float(ref.detach())))
        scale = max(float(p.grad.abs().max()) for p in model.parameters())
        for k, g in res.parameters.items():
            want = dict(model.named_parameters())[k].grad
            if g is not None and g.shape == want.shape:
                err = max(err, float((g - want).abs().max() / scale))
    s = sch.structure
    report = {"grid": {"pp": pp, "cp": cp, "tp": tp}, "processors": len(procs), "by_verb": s["by_verb"],
              "gathering_fallbacks": s["gathering_fallbacks"], "fused": dict(prog.fusion), "signature_ok": sch.signature.ok(),
              "error": err, "ok": bool(err < 2e-4), "compile_s": round(t_compile, 3), "run_s": round(t_run, 4)}
    print(json.dumps(report, default=str), flush=True)
    return report


if __name__ == "__main__":
    main()
