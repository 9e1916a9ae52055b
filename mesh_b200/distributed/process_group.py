"""``torch.distributed`` backend ``"mesh"``.

    import mesh_b200.distributed.process_group   # registers the backend
    dist.init_process_group("mesh", ...)

CUDA tensors are moved by this package's own kernels over the symmetric heap
(:class:`mesh_b200.distributed.comm.Communicator`); CPU tensors are delegated to a gloo group
created over the same store, which is also what the CPU-only tests exercise.  The reference has no
ProcessGroup (its design only mentions an NCCL net plugin that is not in the tree,
design/bridge-and-ipc.md:16-31); the verbs behind this backend are the ones of its verbs table
(design/collective-verbs.md:7-35).

Collectives on CUDA tensors are enqueued on the current stream and the returned ``Work`` is
already complete in the stream-ordered sense, like NCCL's.
"""
from __future__ import annotations

from datetime import timedelta

import torch
import torch.distributed as dist

_REDOP = {dist.ReduceOp.SUM: "sum", dist.ReduceOp.MAX: "max", dist.ReduceOp.MIN: "min",
          dist.ReduceOp.PRODUCT: "prod", dist.ReduceOp.AVG: "avg"}


def _op_name(op) -> str:
    try:
        return _REDOP[op]
    except (KeyError, TypeError):
        for k, v in _REDOP.items():
            if op == k:
                return v
        raise ValueError(f"mesh backend: unsupported reduce op {op}")


class _DoneWork(dist._Work):
    """Completed (stream-ordered) work."""

    def __init__(self, result=None):
        super().__init__()
        self._result = result
        self._fut = None

    def wait(self, timeout=None):
        return True

    def is_completed(self):
        return True

    def is_success(self):
        return True

    def result(self):
        return self._result

    def get_future(self):
        if self._fut is None:
            self._fut = torch.futures.Future()
            self._fut.set_result(self._result)
        return self._fut


class ProcessGroupMesh(dist.ProcessGroup):
    def __init__(self, store, rank: int, world: int, timeout: timedelta | None = None):
        super().__init__(rank, world)
        self._store = store
        self._rank, self._world = rank, world
        self._timeout = timeout or timedelta(seconds=300)
        self._gloo = None
        self._comm = None
        self._heap = None

    # ---------------------------------------------------------------- lazily built halves
    def _cpu(self):
        if self._gloo is None:
            self._gloo = dist.ProcessGroupGloo(dist.PrefixStore("mesh-gloo", self._store), self._rank, self._world,
                                               self._timeout)
        return self._gloo

    def _gpu(self):
        if self._comm is None:
            from ..config import config
            from ..runtime.heap import SymmetricHeap
            from ..runtime.rendezvous import Rendezvous
            from .comm import Communicator
            from .context import current_or_none
            ctx = current_or_none()
            if ctx is not None and ctx.world == self._world and ctx.rank == self._rank and ctx.is_cuda:
                self._heap = ctx.heap
                self._comm = ctx.comm
                return self._comm
            else:
                rdv = Rendezvous(dist.PrefixStore("mesh-heap", self._store), self._rank, self._world,
                                 timeout_s=self._timeout.total_seconds())
                self._heap = SymmetricHeap(rdv, config().heap_bytes, torch.cuda.current_device(),
                                           signal_bytes=config().signal_bytes)
            self._comm = Communicator(self._heap)
        return self._comm

    def getBackendName(self):
        return "mesh"

    def _get_backend_name(self):
        return "mesh"

    @staticmethod
    def _cuda(t) -> bool:
        return (t[0] if isinstance(t, (list, tuple)) else t).is_cuda

    # ---------------------------------------------------------------- collectives
    def allreduce(self, tensors, opts=None):
        if not self._cuda(tensors):
            return self._cpu().allreduce(tensors, opts) if opts is not None else self._cpu().allreduce(tensors)
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        for t in tensors:
            tc = t if t.is_contiguous() else t.contiguous()
            self._gpu().all_reduce(tc, op)
            if tc is not t:
                t.copy_(tc)
        return _DoneWork(tensors)

    def allreduce_coalesced(self, tensors, opts=None):
        return self.allreduce(tensors, opts)

    def broadcast(self, tensors, opts=None):
        if not self._cuda(tensors):
            return self._cpu().broadcast(tensors, opts)
        root = opts.rootRank if opts is not None else 0
        for t in tensors:
            tc = t if t.is_contiguous() else t.contiguous()
            self._gpu().broadcast(tc, root)
            if tc is not t:
                t.copy_(tc)
        return _DoneWork(tensors)

    def reduce(self, tensors, opts=None):
        if not self._cuda(tensors):
            return self._cpu().reduce(tensors, opts)
        for t in tensors:
            self._gpu().reduce(t, opts.rootRank, _op_name(opts.reduceOp))
        return _DoneWork(tensors)

    def allgather(self, output_tensors, input_tensors, opts=None):
        if not self._cuda(input_tensors):
            return self._cpu().allgather(output_tensors, input_tensors, opts) if opts is not None else \
                self._cpu().allgather(output_tensors, input_tensors)
        for outs, inp in zip(output_tensors, input_tensors):
            counts = [o.numel() for o in outs]
            flat = torch.empty(sum(counts), dtype=inp.dtype, device=inp.device)
            self._gpu().all_gather(flat, inp.contiguous(), counts)
            pos = 0
            for o, c in zip(outs, counts):
                o.copy_(flat[pos:pos + c].view_as(o))
                pos += c
        return _DoneWork(output_tensors)

    def _allgather_base(self, output, input, opts=None):
        if not output.is_cuda:
            return self._cpu()._allgather_base(output, input, opts) if opts is not None else \
                self._cpu()._allgather_base(output, input)
        self._gpu().all_gather(output, input.contiguous())
        return _DoneWork(output)

    def allgather_into_tensor_coalesced(self, outputs, inputs, opts=None):
        for o, i in zip(outputs, inputs):
            self._allgather_base(o, i, opts)
        return _DoneWork(outputs)

    def reduce_scatter(self, output_tensors, input_tensors, opts=None):
        if not self._cuda(output_tensors):
            return self._cpu().reduce_scatter(output_tensors, input_tensors, opts)
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        for out, ins in zip(output_tensors, input_tensors):
            counts = [t.numel() for t in ins]
            self._gpu().reduce_scatter(out, torch.cat([t.reshape(-1) for t in ins]), op, counts)
        return _DoneWork(output_tensors)

    def _reduce_scatter_base(self, output, input, opts=None):
        if not output.is_cuda:
            return self._cpu()._reduce_scatter_base(output, input, opts)
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        self._gpu().reduce_scatter(output, input.contiguous(), op)
        return _DoneWork(output)

    def reduce_scatter_tensor_coalesced(self, outputs, inputs, opts=None):
        for o, i in zip(outputs, inputs):
            self._reduce_scatter_base(o, i, opts)
        return _DoneWork(outputs)

    def alltoall_base(self, output, input, output_split_sizes, input_split_sizes, opts=None):
        if not output.is_cuda:
            return self._cpu().alltoall_base(output, input, output_split_sizes, input_split_sizes, opts)
        self._gpu().all_to_all(output, input.contiguous(), list(output_split_sizes) or None, list(input_split_sizes) or None)
        return _DoneWork(output)

    def alltoall(self, output_tensors, input_tensors, opts=None):
        if not self._cuda(output_tensors):
            return self._cpu().alltoall(output_tensors, input_tensors, opts)
        inp = torch.cat([t.reshape(-1) for t in input_tensors])
        out = torch.empty(sum(t.numel() for t in output_tensors), dtype=inp.dtype, device=inp.device)
        self._gpu().all_to_all(out, inp, [t.numel() for t in output_tensors], [t.numel() for t in input_tensors])
        pos = 0
        for t in output_tensors:
            t.copy_(out[pos:pos + t.numel()].view_as(t))
            pos += t.numel()
        return _DoneWork(output_tensors)

    def gather(self, output_tensors, input_tensors, opts=None):
        if not self._cuda(input_tensors):
            return self._cpu().gather(output_tensors, input_tensors, opts)
        root = opts.rootRank
        inp = input_tensors[0].contiguous()
        if self._rank == root:
            flat = torch.empty((self._world, inp.numel()), dtype=inp.dtype, device=inp.device)
            self._gpu().gather(flat, inp, root)
            for r, o in enumerate(output_tensors[0]):
                o.copy_(flat[r].view_as(o))
        else:
            self._gpu().gather(None, inp, root)
        return _DoneWork(output_tensors)

    def scatter(self, output_tensors, input_tensors, opts=None):
        if not self._cuda(output_tensors):
            return self._cpu().scatter(output_tensors, input_tensors, opts)
        root = opts.rootRank
        out = output_tensors[0]
        oc = out if out.is_contiguous() else torch.empty_like(out, memory_format=torch.contiguous_format)
        src = torch.stack([t.reshape(-1) for t in input_tensors[0]]) if self._rank == root else None
        self._gpu().scatter(oc, src, root)
        if oc is not out:
            out.copy_(oc)
        return _DoneWork(output_tensors)

    def send(self, tensors, dst, tag=0):
        if not self._cuda(tensors):
            return self._cpu().send(tensors, dst, tag)
        for t in tensors:
            self._gpu().send(t.contiguous(), dst)
        return _DoneWork(None)

    def recv(self, tensors, src, tag=0):
        if not self._cuda(tensors):
            return self._cpu().recv(tensors, src, tag)
        for t in tensors:
            tc = t if t.is_contiguous() else torch.empty_like(t, memory_format=torch.contiguous_format)
            self._gpu().recv(tc, src)
            if tc is not t:
                t.copy_(tc)
        return _DoneWork(tensors)

    def recv_anysource(self, tensors, tag=0):
        return self._cpu().recv_anysource(tensors, tag)

    def barrier(self, opts=None):
        if torch.cuda.is_available() and self._comm is not None:
            self._comm.barrier()
            return _DoneWork(None)
        return self._cpu().barrier(opts) if opts is not None else self._cpu().barrier()

    def shutdown(self):
        if self._heap is not None and self._comm is not None:
            from .context import current_or_none
            c = current_or_none()
            if c is None or c._heap is not self._heap:
                self._heap.close()
        self._comm = None


def _create(store, rank, world, timeout):
    return ProcessGroupMesh(store, rank, world, timeout)


def register() -> None:
    if "MESH" not in dist.Backend.backend_list and "mesh" not in dist.Backend.backend_list:
        dist.Backend.register_backend("mesh", _create, devices=["cpu", "cuda"])


register()
