"""Binding a compiled program to planned storage and starting it many times.

The reference prepares a compiled program once - its planner lays every value out in an arena (lifetime colouring,
``copies`` sets for executions in flight), ``prepare`` binds the program to that storage, and every execution is one
persistent start, refused as stale once the membership view has moved (compiler/mesh_compiler/bridge.py:71-135,
compiler/mesh_compiler/native.py:1107-1384, rdma/mesh-dataflow.c:287-317, rdma/mesh-collective.c:390).  Here:

* ``workspace(scheduled, copies)`` asks the native planner (``runtime/plan.py::layout``) for the arena of the plan's
  values: what one processor needs at peak when values whose lifetimes do not overlap share bytes, repeated per copy.
* ``Prepared`` owns ``copies`` sets of input buffers (execution ``b`` uses set ``b mod copies``) and starts executions
  through a :class:`~mesh_b200.runtime.plan.Plan`: on one CUDA device with no collective in the plan an execution is the
  launch of a CUDA graph captured once per copy (every address fixed before the run); otherwise it is the executor's
  stream-ordered run.  Either way at most ``horizon`` executions are in flight, ``inputs()`` hands out a set only when the
  execution that last read it has ended, and a start under a newer membership view raises ``MeshStale``.
"""
from __future__ import annotations

from typing import Any

import torch

from . import schedule as _schedule
from .runtime import Program


def workspace(scheduled, copies: int = 1, align: int = 256) -> dict:
    """``{"bytes_per_copy", "bytes_unshared", "copies", "offsets": {value: [offset per copy]}, "transfers": [...],
    "planned": the native planner's demands, order and exposed time for those transfers, "pipeline": its steady state
    for repeated starts (period, latency, copies)}``."""
    from ..runtime.plan import layout
    lt = _schedule.lifetimes(scheduled.plan)
    offs, one = layout([(a, b, c) for _, a, b, c in lt], copies=copies, align=align) if lt else ([[]] * copies, 0)
    return {"bytes_per_copy": one, "bytes_unshared": sum(c for *_, c in lt), "copies": copies,
            "offsets": {name: [offs[c][i] for c in range(copies)] for i, (name, *_rest) in enumerate(lt)},
            "transfers": _schedule.declarations(scheduled.plan), "horizon": _schedule.horizon(scheduled.plan, copies),
            "planned": _schedule.planned(scheduled.plan), "pipeline": _schedule.pipelined(scheduled.plan)}


class Prepared:
    """``prepared = prepare(scheduled, examples)``; ``prepared.inputs()`` -> writable input set of the next execution,
    ``prepared.start()`` -> execution number, ``prepared.result(b)``, ``prepared.ended(b)``, ``prepared.synchronize()``."""

    def __init__(self, scheduled, examples, copies: int | None = 2, horizon: int | None = None, program: Program | None = None,
                 graphs: bool | None = None, rdv=None):
        self.scheduled = scheduled
        self.program = program or Program(scheduled)
        if copies is None:
            # as many sets of buffers as executions are alive at once in the planner's steady state (within reason)
            copies = min(4, max(1, _schedule.pipelined(scheduled.plan)["copies"]))
        self.copies = max(1, copies)
        self.horizon = max(1, min(horizon or self.copies, self.copies))
        dev = self.program.device if isinstance(self.program.device, torch.device) else torch.device("cpu")
        self.device = dev
        self._inputs = [[e.detach().clone().to(dev) if torch.is_tensor(e) else e for e in examples] for _ in range(self.copies)]
        self.plan_info = workspace(scheduled, self.copies)
        has_collectives = any(st.op in ("collective", "fused") and "channel" in st.meta for st in self.program.plan.steps)
        graphable = dev.type == "cuda" and self.program.threads and self.program.mesh.size == 1 and not has_collectives
        self.graphs = graphable if graphs is None else (graphs and graphable)
        if rdv is None:
            from ..distributed.context import current_or_none
            ctx = current_or_none()
            rdv = ctx.rdv if ctx is not None else None
        self.rdv = rdv
        self.epoch = rdv.epoch if rdv is not None else 0
        self._results: dict[int, Any] = {}
        self._static: list = [None] * self.copies
        self._events: dict[int, Any] = {}
        self.started = 0
        self._plan = None
        if self.graphs:
            from ..runtime.plan import Plan
            self._plan = Plan(rdv, copies=self.copies, horizon=self.horizon)
            for c in range(self.copies):
                self._plan.capture(c, lambda c=c: self._static.__setitem__(c, self.program(*self._inputs[c])))

    # ---- the reference's runner surface
    def ended(self, execution: int | None = None) -> bool:
        b = self.started - 1 if execution is None else execution
        if b < 0 or b >= self.started:
            return b < 0
        ev = self._events.get(b)
        return True if ev is None else bool(ev.query())

    def inputs(self):
        """The input set of the next execution; waits until the execution that last read it has ended."""
        b = self.started
        prev = b - self.copies
        if prev >= 0 and not self.ended(prev):
            self._events[prev].synchronize()
        return self._inputs[b % self.copies]

    def start(self, *args) -> int:
        """Start the next execution (optionally after copying ``args`` into its input set).  Returns its number."""
        if self.rdv is not None:
            self.rdv.check_epoch(self.epoch)
        b = self.started
        c = b % self.copies
        oldest = b - self.horizon
        if oldest >= 0 and not self.ended(oldest):
            self._events[oldest].synchronize()
        if args:
            for dst, src in zip(self.inputs(), args):
                if torch.is_tensor(dst):
                    dst.copy_(src, non_blocking=True)
        if self._plan is not None:
            self._plan.start()
            out = self._static[c]
        else:
            out = self.program(*self._inputs[c])
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._events[b] = ev
        self._results[b] = out
        self._results.pop(b - self.copies, None)
        self._events.pop(b - 2 * self.copies, None)
        self.started += 1
        return b

    def result(self, execution: int | None = None):
        """The outputs of ``execution`` (default: the latest); with graphs they live in that copy's static storage
        and are overwritten ``copies`` executions later."""
        b = self.started - 1 if execution is None else execution
        if b not in self._results:
            raise KeyError(f"execution {b} is no longer held (copies = {self.copies})")
        ev = self._events.get(b)
        if ev is not None:
            ev.synchronize()
        return self._results[b]

    def synchronize(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def retire(self) -> None:
        self.synchronize()
        if self._plan is not None:
            self._plan.retire()
        self._results.clear()


def prepare(scheduled, examples, copies: int | None = 2, horizon: int | None = None, **kw) -> Prepared:
    return Prepared(scheduled, examples, copies, horizon, **kw)
