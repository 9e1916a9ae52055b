"""Pipeline parallelism: one-forward-one-backward schedule over point-to-point sends (NCCL on GPUs, gloo on CPU).

The reference pipelines by placing layers on different processors, whose crossing edges become send/recv
(examples/engines.py:91-96), and by keeping several executions of a plan in flight (``copies`` / ``horizon``,
rdma/mesh-flow.c:7-12); it names no training schedule.  This module adds the usual one: stage ``s`` of ``P`` runs
``P - s - 1`` warm-up forwards, then alternates one forward with one backward, then drains the backwards, so at most
``P - s`` microbatches of activations are alive on a stage.  A send toward a neighbour and the receive of the
opposite direction from the same neighbour are issued as one batch, which is what keeps two stages that both want
to send first from waiting on each other.

On GPUs the transfers overlap the compute (``_AsyncWire``): activations and gradients travel on two communicators of
their own, every send is issued as soon as its tensor has been computed and is not waited for, and every receive is
posted one phase ahead, so that the next microbatch's input arrives during the current backward pass and the next
gradient during the current forward pass; the compute stream waits (on the device, not the host) only where it first
reads a received tensor.  ``MESH_PP_OVERLAP=0`` goes back to the batched, waited exchanges.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist


class _Wire:
    """Batched point-to-point along the pipeline axis."""

    def __init__(self, axis):
        self.axis = axis
        self.prev = None if axis.first else axis.peer(-1)
        self.next = None if axis.last else axis.peer(+1)
        self.sent_bytes = 0

    def exchange(self, send_prev=None, send_next=None, recv_prev=None, recv_next=None):
        ops = []
        g = self.axis.group
        for t, peer, fn in ((send_prev, self.prev, dist.isend), (recv_prev, self.prev, dist.irecv),
                            (send_next, self.next, dist.isend), (recv_next, self.next, dist.irecv)):
            if t is not None and peer is not None:
                ops.append(dist.P2POp(fn, t, peer, group=g))
                if fn is dist.isend:
                    self.sent_bytes += t.numel() * t.element_size()
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()


class _AsyncWire:
    """Point-to-point along the pipeline axis without waits on the critical path (NCCL ranks).

    Two communicators: ``axis.group`` carries activations toward later stages, ``axis.group_back`` gradients toward
    earlier ones.  Sends are queued on a side stream and never waited for on the compute stream (the sender goes on
    while the next stage is still busy); on each communicator this rank's operations are queued in the order of the
    data flow, which is the order the neighbours use too."""

    def __init__(self, axis):
        self.axis = axis
        self.prev = None if axis.first else axis.peer(-1)
        self.next = None if axis.last else axis.peer(+1)
        self.sent_bytes = 0
        self.sends: list = []          # (work, tensor): kept until the end of the step
        self.side = torch.cuda.Stream(axis.device)
        self._connect()

    def _connect(self):
        """First use of the axis: one blocking word along every link in both directions, pair by pair from the first
        stage on.  NCCL creates the communicator of a pair of ranks at their first transfer, and that creation blocks
        the host until both ranks are in it; the schedule below posts a stage's receive of gradients before the later
        stage can send any, so without this step the first stage would wait for the creation on the gradient
        communicator while the second waits for it on the activation communicator."""
        axis = self.axis
        if getattr(axis, "_pp_connected", False):
            return
        t = torch.zeros(1, device=axis.device)
        for r in range(axis.world - 1):
            if axis.rank == r:
                dist.send(t, self.next, group=axis.group)
                dist.recv(t, self.next, group=axis.group_back)
            elif axis.rank == r + 1:
                dist.recv(t, self.prev, group=axis.group)
                dist.send(t, self.prev, group=axis.group_back)
        torch.cuda.synchronize(axis.device)
        axis._pp_connected = True

    def _post(self, fn, t, peer, group):
        main = torch.cuda.current_stream(self.axis.device)
        self.side.wait_stream(main)                  # the tensor (a send's payload, a receive's buffer) exists
        with torch.cuda.stream(self.side):
            w = fn(t, peer, group=group)
        t.record_stream(self.side)
        return w

    def send_next(self, t):
        if self.next is not None:
            self.sent_bytes += t.numel() * t.element_size()
            self.sends.append((self._post(dist.isend, t, self.next, self.axis.group), t))

    def send_prev(self, t):
        if self.prev is not None and t is not None:
            self.sent_bytes += t.numel() * t.element_size()
            self.sends.append((self._post(dist.isend, t, self.prev, self.axis.group_back), t))

    def recv_prev(self, buf):
        return None if self.prev is None else (self._post(dist.irecv, buf, self.prev, self.axis.group), buf)

    def recv_next(self, buf):
        return None if self.next is None else (self._post(dist.irecv, buf, self.next, self.axis.group_back), buf)

    @staticmethod
    def take(posted):
        """The received tensor; the current stream waits for its arrival."""
        if posted is None:
            return None
        w, buf = posted
        w.wait()
        return buf

    def drain(self):
        for w, _ in self.sends:
            w.wait()
        self.sends.clear()


def _overlapped(axis) -> bool:
    """Asynchronous sends from the second step of an axis on: the first step runs with matched, waited transfers, so
    that every kernel of the step has been launched once (loading a module can make the host wait for the device, which
    must not happen while a send that the next stage has not asked for yet is running)."""
    import os
    return (os.environ.get("MESH_PP_OVERLAP", "1") != "0" and axis.device.type == "cuda"
            and getattr(axis, "group_back", None) is not None and axis.world > 1 and getattr(axis, "_pp_warm", False))


def run_1f1b(stage: Callable[[torch.Tensor], torch.Tensor], axis, microbatches: Sequence, *,
             act_shape: Sequence[int], act_dtype: torch.dtype, loss_fn: Callable | None = None,
             targets: Sequence | None = None, grad_scale: float | None = None):
    """Run one training step of a pipeline stage.

    ``stage(x)`` maps the activations received from the previous stage (on the first stage: the microbatch itself)
    to the activations for the next one.  On the last stage ``loss_fn(y, target)`` turns them into a scalar; its
    gradient is scaled by ``grad_scale`` (default ``1 / len(microbatches)``), so parameter gradients come out as the
    mean over microbatches.  ``microbatches`` must have the same length on every stage (only the first stage reads
    the entries).  Returns the list of microbatch losses on the last stage (``[]`` elsewhere) and statistics.
    """
    M = len(microbatches)
    P, s = axis.world, axis.rank
    wire = _Wire(axis)
    scale = 1.0 / M if grad_scale is None else grad_scale
    dev = axis.device
    warm = min(P - s - 1, M)
    rem = M - warm
    alive: list[tuple] = []            # (input, output) of forwards whose backward has not run
    losses: list[torch.Tensor] = []
    peak_alive = 0

    def new_act():
        return torch.empty(tuple(act_shape), dtype=act_dtype, device=dev)

    def forward(i: int, x_in):
        nonlocal peak_alive
        if axis.first:
            x = microbatches[i]
        else:
            x = x_in.requires_grad_(True)
        y = stage(x)
        if axis.last:
            if loss_fn is None:
                raise ValueError("the last stage needs loss_fn")
            loss = loss_fn(y, None if targets is None else targets[i])
            losses.append(loss.detach())
            y = loss
        alive.append((x, y))
        peak_alive = max(peak_alive, len(alive))
        return y

    def backward(gy):
        x, y = alive.pop(0)
        if axis.last:
            (y * scale).backward()
        else:
            torch.autograd.backward(y, gy)
        if axis.first:
            return None
        g = x.grad
        x.grad = None
        return g

    if _overlapped(axis):
        # Same schedule, sends off the critical path: see _AsyncWire.  A receive is posted where its data is needed, not
        # earlier: an NCCL receive is a kernel that runs until its sender arrives, and whatever makes the host wait for
        # the whole device meanwhile (a module loaded at a kernel's first launch, a freed block) would then wait for a
        # peer that may be waiting for this rank.
        aw = _AsyncWire(axis)
        n_fwd = n_bwd = 0

        def do_forward():
            nonlocal n_fwd
            x_in = None if axis.first else aw.take(aw.recv_prev(new_act()))
            y = forward(n_fwd, x_in)
            n_fwd += 1
            if not axis.last:
                aw.send_next(y.detach())

        def do_backward():
            nonlocal n_bwd
            gy = None if axis.last else aw.take(aw.recv_next(new_act()))
            gx = backward(gy)
            n_bwd += 1
            aw.send_prev(gx)

        for _ in range(warm):
            do_forward()
        for _ in range(rem):
            do_forward()
            do_backward()
        for _ in range(warm):
            do_backward()
        aw.drain()
        return losses, {"peak_alive": peak_alive, "sent_bytes": aw.sent_bytes, "microbatches": M, "overlapped": True}
    # ---- warm-up forwards
    for i in range(warm):
        x_in = None
        if not axis.first:
            x_in = new_act()
            wire.exchange(recv_prev=x_in)
        y = forward(i, x_in)
        wire.exchange(send_next=None if axis.last else y.detach())
    # ---- steady state
    x_in = None
    if rem > 0 and not axis.first:
        x_in = new_act()
        wire.exchange(recv_prev=x_in)
    for i in range(rem):
        y = forward(warm + i, x_in)
        gy = None
        if not axis.last:
            gy = new_act()
            wire.exchange(send_next=y.detach(), recv_next=gy)
        gx = backward(gy)
        if i + 1 < rem:
            x_in = None if axis.first else new_act()
            wire.exchange(send_prev=gx, recv_prev=x_in)
        else:
            wire.exchange(send_prev=gx)
    # ---- drain
    for _ in range(warm):
        gy = None
        if not axis.last:
            gy = new_act()
            wire.exchange(recv_next=gy)
        gx = backward(gy)
        wire.exchange(send_prev=gx)
    try:
        axis._pp_warm = True
    except AttributeError:
        pass
    return losses, {"peak_alive": peak_alive, "sent_bytes": wire.sent_bytes, "microbatches": M}


def split_layers(n_layers: int, stages: int) -> list[range]:
    """Contiguous layer ranges per stage, earlier stages taking the remainder."""
    base, extra = divmod(n_layers, stages)
    out, lo = [], 0
    for s in range(stages):
        n = base + (1 if s < extra else 0)
        out.append(range(lo, lo + n))
        lo += n
    return out
