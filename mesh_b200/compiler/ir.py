"""Intermediate representation of the sharding compiler.

* ``mesh::send(value, channel)`` / ``mesh::recv(channel)``: custom ops with *eager* semantics — a
  per-thread table of queues — so that a scheduled program can be interpreted with one thread per
  processor and plain torch ops (the reference's counterfactual program, compiler/mesh_compiler/ir.py:20-42,
  design/data-flow.md:67-160).  The interpreter is both the bring-up executor and the oracle for
  programs that later run one process per GPU.
* ``Spec``: placement of a value along one axis of the processor mesh — replicated, sharded along a
  tensor dimension (equal, unequal or striped), a pending partial reduction, or whole on one processor.
* ``Step`` / ``Plan``: the SPMD program every processor runs, with its collectives made explicit
  (kind ``broadcast`` | ``reduce`` | ``alltoall`` | ``permute``, compiler/mesh_compiler/placement.py:946-953).
* ``Scheduled``: what ``compile_module`` returns and ``Program`` runs; ``TrainingResult`` is the pytree a
  joint forward+backward program returns (compiler/mesh_compiler/ir.py:79-84).
"""
from __future__ import annotations

import dataclasses
import queue
import threading
from typing import Any, NamedTuple

import torch

def pack(*items) -> tuple:
    """Step target: the values of several steps as one tuple (an operator's results put back together)."""
    return tuple(items)


JOIN, PAGES = "join", "pages"       # consumers of a transfer: wait for all of it / take pieces as they land

# ----------------------------------------------------------------------------- eager send / recv
LOCAL = threading.local()


class Channels:
    """Queues shared by the threads of one interpreted program."""

    def __init__(self):
        self._lock = threading.Lock()
        self._q: dict[Any, queue.Queue] = {}

    def get(self, key) -> queue.Queue:
        with self._lock:
            q = self._q.get(key)
            if q is None:
                q = self._q[key] = queue.Queue()
            return q


def _channels() -> Channels:
    ch = getattr(LOCAL, "channels", None)
    if ch is None:
        ch = LOCAL.channels = Channels()
    return ch


_lib = torch.library.Library("mesh", "DEF")
_lib.define("send(Tensor value, int channel) -> ()")
_lib.define("recv(int channel) -> Tensor")


@torch.library.impl(_lib, "send", "CompositeExplicitAutograd")
def _send(value, channel):
    _channels().get(channel).put(value.detach())


@torch.library.impl(_lib, "recv", "CompositeExplicitAutograd")
def _recv(channel):
    return _channels().get(channel).get(timeout=getattr(LOCAL, "timeout", 60.0))


try:  # ordered effects: send/recv are never reordered or dropped by export passes
    from torch._higher_order_ops.effects import _EffectType, _register_effectful_op
    _register_effectful_op(torch.ops.mesh.send.default, _EffectType.ORDERED)
    _register_effectful_op(torch.ops.mesh.recv.default, _EffectType.ORDERED)
except Exception:  # pragma: no cover - private API moved; eager semantics do not depend on it
    pass

send = torch.ops.mesh.send
recv = torch.ops.mesh.recv


# ----------------------------------------------------------------------------- placements
@dataclasses.dataclass(frozen=True)
class Spec:
    """Placement along ONE mesh axis."""
    kind: str = "R"                 # R replicated | S sharded | P partial (pending reduction) | O whole on one owner
    dim: int = -1                   # S: tensor dimension
    counts: tuple = ()              # S: elements of `dim` held by each processor of the axis
    striped: bool = False           # S: processor j holds elements j, j+P, ... (equal counts reduce to P*i + j)
    owner: int = -1                 # O: index along the axis
    op: str = "sum"                 # P: pending reduction

    def __repr__(self):
        if self.kind == "S":
            return f"S({self.dim}{',striped' if self.striped else ''},{list(self.counts)})"
        if self.kind == "O":
            return f"O({self.owner})"
        return self.kind


R = Spec("R")


def S(dim: int, counts, striped: bool = False) -> Spec:
    return Spec("S", dim, tuple(int(c) for c in counts), striped)


def P(op: str = "sum") -> Spec:
    return Spec("P", op=op)


def O(owner: int) -> Spec:
    return Spec("O", owner=owner)


class Mesh(NamedTuple):
    """Processor grid: ``shape`` per axis, ``names`` in row-major order (``names[i]`` is rank i)."""
    names: tuple
    shape: tuple

    @property
    def size(self) -> int:
        return len(self.names)

    def coords(self, rank: int) -> tuple:
        out, r = [], rank
        for s in reversed(self.shape):
            out.append(r % s)
            r //= s
        return tuple(reversed(out))

    def axis_group(self, rank: int, axis: int) -> tuple:
        """Ranks that differ from ``rank`` only along ``axis`` (in axis order)."""
        c = list(self.coords(rank))
        out = []
        for i in range(self.shape[axis]):
            c[axis] = i
            r = 0
            for s, v in zip(self.shape, c):
                r = r * s + v
            out.append(r)
        return tuple(out)


@dataclasses.dataclass
class Step:
    """One instruction of the SPMD plan.

    ``op``: ``"call"`` (run ``target`` on local values) | ``"collective"`` | ``"slice"`` (local narrow of a
    replicated value) | ``"const"``.  ``args`` reference earlier values by name (``Ref``).
    """
    op: str
    out: str
    target: Any = None
    args: tuple = ()
    kwargs: dict = dataclasses.field(default_factory=dict)
    meta: dict = dataclasses.field(default_factory=dict)


class Ref(NamedTuple):
    name: str


@dataclasses.dataclass
class Transfer:
    """A collective the compiler inserted (what the structure report counts)."""
    channel: int
    kind: str            # broadcast | reduce | alltoall | permute
    verb: str            # all_gather | all_reduce | reduce_scatter | all_to_all | send_recv | slice
    axis: int
    value: str
    dimension: int
    counts: tuple
    consumer: str = JOIN
    nbytes: int = 0


@dataclasses.dataclass
class Plan:
    mesh: Mesh
    steps: list
    inputs: list                     # placeholder names in call order
    input_specs: dict                # name -> tuple[Spec] (how the caller's full tensor is cut)
    outputs: list                    # (name | constant) per flat output
    output_specs: dict
    transfers: list
    full_shapes: dict                # name -> global shape
    dtypes: dict
    duplicated: int = 0              # invariant values recomputed where they are read instead of transferred


@dataclasses.dataclass
class Exported:
    graph_module: torch.fx.GraphModule
    state: dict                      # placeholder name -> (qualified name, tensor) for parameters / buffers / constants
    state_kinds: dict                # placeholder name -> "parameter" | "buffer" | "constant"
    user_inputs: list                # placeholder names of user inputs, in order
    outputs: list                    # (kind, target) per flat graph output: "user" | "loss" | "grad_param" | "grad_input" | "mutation"
    in_spec: Any
    out_spec: Any
    mutations: dict                  # output index -> placeholder name written in place
    training: bool = False
    program: Any = None              # the torch.export.ExportedProgram (what archives store)
    tied: dict = dataclasses.field(default_factory=dict)    # parameter name -> the name it shares its tensor with


class TrainingResult(NamedTuple):
    outputs: Any
    parameters: dict
    inputs: dict


@dataclasses.dataclass
class Scheduled:
    exported: Exported
    plan: Plan
    processors: dict
    placement_repr: dict             # node name -> stated placement (for archives / reports)
    signature: Any = None            # ordered synchronisation operations + static check result
    structure: dict = dataclasses.field(default_factory=dict)
    output_processor: str | None = None
    cost: Any = None
