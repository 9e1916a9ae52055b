"""The older one-call interface: ``program(block, *examples)`` -> ``run``, with ``Placement`` / ``Shard`` records.

The reference still documents this surface as its torch binding (rdma/mesh_compile.py: ``Placement(mesh, nodes,
splits)`` :43, ``Shard(m, units)`` :62, ``Function`` :7785, ``program`` :8364, runner attributes :8777-8831, ``load``
:8744).  Here it is a thin layer over the compiler proper: ``program`` compiles the block (or a program of
``Function`` leaves compiled once and called many times) and returns a runner that owns ``copies`` sets of input
buffers; execution ``b`` reads set ``b mod copies``, and ``run.inputs()`` hands out the next set once execution
``b - horizon`` has ended, which is how a caller keeps several executions in flight without overwriting inputs that
are still being read (rdma/mesh-flow.c:7-12).
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass, field
from typing import Any

import torch

from . import archive
from .driver import compile_module, compile_program
from .runtime import Program


@dataclass(frozen=True)
class Shard:
    """Cut dimension ``m`` into shares ``units`` (``None``: equal chunks; ratios; ``"striped"``)."""
    m: int
    units: Any = None


@dataclass
class Placement:
    """``mesh``: processor names in order; ``nodes``: ``{glob pattern over graph node names: split key or processor
    name}``; ``splits``: ``{key: Shard}``.  Calling it with a graph node gives what the compiler's placement
    callables return."""
    mesh: tuple
    nodes: dict = field(default_factory=dict)
    splits: dict = field(default_factory=dict)

    def __call__(self, node):
        if node.op not in ("placeholder", "call_function", "get_attr"):
            return None
        for pattern, what in self.nodes.items():
            if fnmatch.fnmatchcase(node.name, pattern):
                if what in self.splits:
                    sh = self.splits[what]
                    return (sh.m, tuple(self.mesh), sh.units)
                if what in self.mesh:
                    return what
                raise KeyError(f"placement of {node.name!r}: {what!r} is neither a split nor a processor")
        return None


class Function(torch.nn.Module):
    """Marks ``module`` as a function of the program: compiled once, called as often as the block calls it.
    ``weights`` optionally replaces the module's state before compilation (name -> tensor)."""

    def __init__(self, module: torch.nn.Module, placement: Placement | None = None, weights: dict | None = None):
        super().__init__()
        self.body, self.placement = module, placement
        if weights:
            module.load_state_dict(weights, strict=False)

    def forward(self, *args, **kwargs):
        return self.body(*args, **kwargs)


class _Runner:
    """The runner of the older interface over :class:`~mesh_b200.compiler.bridge.Prepared`: ``copies`` input sets,
    at most ``horizon`` executions in flight, executions started on the device's stream (one CUDA-graph launch each
    where the program allows it) and their ends observed through events."""

    def __init__(self, scheduled, examples, copies: int, horizon: int):
        from .bridge import Prepared
        self.scheduled, self.copies = scheduled, max(1, copies)
        self._prepared = Prepared(scheduled, examples, copies=self.copies, horizon=max(1, horizon))
        self.horizon = self._prepared.horizon
        self._program = self._prepared.program

    # -- attributes of the reference's runner
    @property
    def signature(self):
        return self.scheduled.signature

    @property
    def structure(self):
        return self.scheduled.structure

    @property
    def results(self) -> dict:
        return self._prepared._results

    @property
    def _inputs(self):
        return self._prepared._inputs

    def ended(self, execution: int | None = None) -> bool:
        """Whether ``execution`` (default: the latest started) has finished."""
        return self._prepared.ended(execution)

    def inputs(self):
        """The writable input set of the next execution; waits until the execution that last used it is over."""
        return self._prepared.inputs()

    def __call__(self, *args):
        b = self._prepared.start(*args)
        return self._prepared._results[b]

    def synchronize(self) -> None:
        self._prepared.synchronize()

    def save(self, directory: str) -> None:
        archive.save(directory, self.scheduled)
        torch.save({"examples": self._inputs[0], "copies": self.copies, "horizon": self.horizon}, f"{directory}/runner.pt")


def program(block: torch.nn.Module, *examples, processors: dict, placement=None, copies: int = 2, horizon: int = 1,
            **export_options) -> _Runner:
    """Compile ``block`` for ``examples`` and return its runner.  Submodules wrapped in :class:`Function` are compiled
    once each; a ``Function``'s own placement overrides the program's for the nodes it matches."""
    leaves = {name: m for name, m in block.named_modules() if isinstance(m, Function)}
    placements = [m.placement for m in leaves.values() if m.placement is not None]

    def place(node):
        for p in placements:
            got = p(node)
            if got is not None:
                return got
        return placement(node) if placement is not None else None
    if leaves:
        sch = compile_program(block, examples, set(leaves), processors, place, **export_options)
    else:
        sch = compile_module(block, examples, processors, place, **export_options)
    return _Runner(sch, examples, copies, horizon)


def load(directory: str) -> _Runner:
    """The runner of a program saved with ``run.save``."""
    meta = torch.load(f"{directory}/runner.pt", weights_only=False)
    return _Runner(archive.load(directory), meta["examples"], meta["copies"], meta["horizon"])
