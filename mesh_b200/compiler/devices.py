"""Processors onto devices, and the transfers that cross between machines.

A processor is described as ``(machine, device)``.  The reference's ``on_devices`` stage puts every node of the placed
graph on its processor's torch device and inserts a copy wherever a value crosses (compiler/mesh_compiler/devices.py:
22-72).  Here the plan is one program for all processors, so the devices are a property of the run, not of the graph:
``Program(scheduled, device="processors")`` interprets the plan with one thread per processor, each on the device its
description names, and a value that arrives from another processor is copied to the receiver's device where it lands.
With one process per GPU the question does not come up (every rank computes on its own GPU and the collectives move
the data), and the engines that are not GPUs are reached through ``mesh_b200.runtime.host_engine``.

:func:`crossings` is the accounting half: which of the compiled transfers have members on more than one machine (or
device), and how many bytes they move - the "between machines" figure of the examples' reports.
"""
from __future__ import annotations

import torch

from .ir import Plan


ENGINES = ("host",)       # device names that are engines of this package rather than torch devices


def is_engine(description) -> bool:
    """Is the processor an engine that is not a torch device?  ``"host"``: the host engine
    (``mesh_b200.runtime.host_engine``), the counterpart of the reference's processors that are neither CPU nor GPU
    code paths of torch (its ``'ane'`` device, compiler/mesh_compiler/devices.py:50-69, lower_coreml.py:101-321): the
    products, norms and sums placed there run as batches on the engine's own threads over host memory, and the
    engine reports which device ran each of them."""
    name = description[1] if isinstance(description, (tuple, list)) else description
    return str(name) in ENGINES


def device_of(description, available_only: bool = False) -> torch.device:
    """The torch device of one processor description ``(machine, device)`` (or a bare device); an engine's values
    live in host memory."""
    name = description[1] if isinstance(description, (tuple, list)) else description
    if str(name) in ENGINES:
        return torch.device("cpu")
    dev = torch.device(name)
    if dev.type == "cuda" and available_only and not torch.cuda.is_available():
        return torch.device("cpu")
    return dev


def on_devices(processors: dict, available_only: bool = True) -> list[torch.device]:
    """One device per processor, in rank order.  ``available_only`` maps CUDA devices to the CPU on a host without a
    GPU, so that a program compiled for GPUs can still be interpreted there."""
    return [device_of(d, available_only) for d in processors.values()]


def crossings(plan: Plan, processors: dict) -> dict:
    """Transfers whose participants are on more than one machine / device.

    Returns ``{"transfers", "between_machines", "between_devices", "bytes_between_machines", "bytes_between_devices",
    "by_kind"}``; bytes are the transfer's declared size, counted once per transfer."""
    names = list(processors)
    machines = [processors[n][0] if isinstance(processors[n], (tuple, list)) else 0 for n in names]
    devices = [(m, str(device_of(processors[n]))) for m, n in zip(machines, names)]
    mesh = plan.mesh
    out = {"transfers": len(plan.transfers), "between_machines": 0, "between_devices": 0,
           "bytes_between_machines": 0, "bytes_between_devices": 0, "by_kind": {}}
    for t in plan.transfers:
        groups = {mesh.axis_group(r, t.axis) for r in range(mesh.size)}
        over_machines = any(len({machines[r] for r in g}) > 1 for g in groups)
        over_devices = any(len({devices[r] for r in g}) > 1 for g in groups)
        if over_machines:
            out["between_machines"] += 1
            out["bytes_between_machines"] += t.nbytes
            out["by_kind"][t.kind] = out["by_kind"].get(t.kind, 0) + 1
        if over_devices:
            out["between_devices"] += 1
            out["bytes_between_devices"] += t.nbytes
    return out
