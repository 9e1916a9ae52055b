"""Per-process runtime context: one process per GPU.

``init()`` is the counterpart of the reference's ``mesh_attach`` (rdma/mesh-dataflow.c:40): it joins
the rank table, brings up peer mappings (the symmetric heap) and hands back the object every layer
and collective hangs off.  ``shutdown()`` is the bounded, ordered teardown (``mesh_detach``).
"""
from __future__ import annotations

import os
from datetime import timedelta

import torch
import torch.distributed as dist

from ..config import config
from ..runtime.rendezvous import Rendezvous

_ctx: "MeshContext | None" = None


class MeshContext:
    def __init__(self, rank: int, world: int, device: torch.device, rdv: Rendezvous, group=None):
        self.rank, self.world, self.device, self.rdv, self.group = rank, world, device, rdv, group
        self._heap = None
        self.launches = 0          # kernels of this library launched (bench accounting)

    @property
    def heap(self):
        """Symmetric heap, created on first use (CUDA only)."""
        if self._heap is None:
            from ..runtime.heap import SymmetricHeap
            cfg = config()
            self._heap = SymmetricHeap(self.rdv, cfg.heap_bytes, self.device.index, signal_bytes=cfg.signal_bytes,
                                       multicast=cfg.nvls and self.world > 1 and os.environ.get("MESH_NVLS", "0") == "1")
        return self._heap

    @property
    def comm(self):
        """This context's Communicator (collective kernels over the heap), created on first use."""
        if getattr(self, "_comm", None) is None:
            from .comm import Communicator
            self._comm = Communicator(self.heap)
        return self._comm

    @property
    def is_cuda(self) -> bool:
        return self.device.type == "cuda"


def init(backend: str | None = None, device: str | torch.device | None = None, timeout_s: float = 120.0) -> MeshContext:
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (torchrun) or run solo.

    ``backend``: the torch.distributed backend used for plumbing (barriers, object exchange, pipeline
    p2p): ``"nccl"`` on GPUs, ``"gloo"`` on CPU, or ``"mesh"`` for this package's own backend.
    """
    global _ctx
    if _ctx is not None:
        return _ctx
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if device is None:
        device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    device = torch.device(device)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if backend is None:
        backend = "nccl" if device.type == "cuda" else "gloo"
    group = None
    if world > 1 or "MASTER_ADDR" in os.environ:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if not dist.is_initialized():
            kw = {"device_id": device} if (backend == "nccl") else {}
            dist.init_process_group(backend, rank=rank, world_size=world, timeout=timedelta(seconds=timeout_s), **kw)
        group = dist.group.WORLD
        from torch.distributed import distributed_c10d as c10d
        store = dist.PrefixStore("mesh_b200", c10d._get_default_store())
    else:
        store = dist.HashStore()
    rdv = Rendezvous(store, rank, world, timeout_s=timeout_s)
    _ctx = MeshContext(rank, world, device, rdv, group)
    return _ctx


def current_or_none() -> "MeshContext | None":
    return _ctx


def context() -> MeshContext:
    if _ctx is None:
        return init()
    return _ctx


def shutdown() -> None:
    global _ctx
    if _ctx is None:
        return
    if _ctx._heap is not None:
        _ctx._heap.close()
    if dist.is_initialized():
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()
    _ctx = None
