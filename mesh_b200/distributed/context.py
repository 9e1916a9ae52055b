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
        self.monitor = None        # ErrorMonitor of this process's device (CUDA only)
        self.service = False       # runtime service (stats block + heartbeat thread) running

    @property
    def heap(self):
        """Symmetric heap, created on first use (CUDA only)."""
        if self._heap is None:
            from ..runtime.heap import SymmetricHeap
            cfg = config()
            self._heap = SymmetricHeap(self.rdv, cfg.heap_bytes, self.device.index, signal_bytes=cfg.signal_bytes,
                                       multicast=cfg.nvls and self.world > 1 and os.environ.get("MESH_NVLS", "0") == "1")
            if self.service:
                from ..runtime import service
                for peer in range(min(self.world, 8)):                   # every peer's segment is mapped: the channel is up
                    service.channel(peer, "CONNECTED")
        return self._heap

    @property
    def comm(self):
        """This context's Communicator (collective kernels over the heap), created on first use."""
        if getattr(self, "_comm", None) is None:
            from .comm import Communicator
            self._comm = Communicator(self.heap)
        return self._comm

    @property
    def channels(self):
        """Peer channels of this process (``runtime/channels.py``): created with the heap, one per peer, CONNECTED
        once the peers' segments are mapped.  They carry the transfers that are left to the copy engines."""
        if getattr(self, "_channels", None) is None:
            from ..runtime.channels import PeerChannels
            _ = self.heap                                   # peers are mapped first
            self._channels = PeerChannels(self.rank, self.world, self.device.index if self.is_cuda else -1)
            self._channels.connect_all()
        return self._channels

    def bulk_put(self, dst, peer: int, src: torch.Tensor) -> int:
        """Store ``src`` into rank ``peer``'s copy of the symmetric buffer ``dst`` with the copy engines (no SM is
        used), ordered after the work now on the current stream.  Returns a ticket for ``channels.done`` /
        ``channels.wait_on_stream``.  For bulk moves (re-sharding, weight distribution at start-up); the collectives and
        the fused layers move their data from inside kernels."""
        n = src.numel() * src.element_size()
        if n > dst.nbytes:
            raise ValueError("bulk_put: source larger than the destination buffer")
        stream = torch.cuda.current_stream(self.device).cuda_stream if self.is_cuda else 0
        return self.channels.copy(peer, dst.ptr(peer), src.data_ptr(), n, stream)

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
    _start_runtime(_ctx)
    return _ctx


def _start_runtime(ctx: "MeshContext") -> None:
    """The per-process runtime that every job gets: the stats block with its heartbeat thread (what ``meshctl status``
    and ``meshctl top`` read, and what a supervisor watches) and, on a GPU, the error monitor that spreads the abort
    flag after the first device-side failure.  ``MESH_RUNTIME=0`` leaves both out (a process that must not start
    threads).  A missing native library on a CPU-only machine leaves them out too."""
    if os.environ.get("MESH_RUNTIME", "1") == "0":
        return
    from .. import _native
    cfg = config()
    try:
        from ..runtime import service
        service.start(cfg.group, ctx.rank, ctx.world, cfg.heartbeat_s)
        service.count("epoch", ctx.rdv.epoch)
        if cfg.deadline_s > 0:
            service.deadline(cfg.deadline_s)
        ctx.service = True
        _native.on_launch = lambda n: service.count("launches", n)
    except Exception:
        ctx.service = False
    if ctx.is_cuda:
        try:
            from ..runtime.monitor import ErrorMonitor
            ctx.monitor = ErrorMonitor(ctx.device)
        except Exception:
            ctx.monitor = None


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
    # in order: the monitor stops reading status blocks, the heap drains and unmaps, the service says goodbye last
    if _ctx.monitor is not None:
        _ctx.monitor.stop()
        _ctx.monitor = None
    if getattr(_ctx, "_channels", None) is not None:
        _ctx._channels.close()                              # bounded flush, proxy thread joined, channels CLOSED
        _ctx._channels = None
    if _ctx._heap is not None:
        _ctx._heap.close()
    if _ctx.service:
        from .. import _native
        from ..runtime import service
        _native.on_launch = None
        service.stop(unlink=True)
        _ctx.service = False
    if dist.is_initialized():
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()
    _ctx = None
