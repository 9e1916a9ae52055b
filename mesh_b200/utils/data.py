"""Input pipeline pieces.  ``DevicePrefetcher`` keeps the host-to-device copy of the next step's input off the
critical path: copies run on a side stream into a small ring of device buffers while the current step computes."""
from __future__ import annotations

from typing import Callable, Iterable, Iterator

import torch


class DevicePrefetcher:
    """``next()`` returns the device copy of the next host batch and at once starts copying the one after it.

    ``source``: an iterable of pinned host tensors (or a callable returning the next one).  The copy of batch ``i + 1``
    is ordered after everything that was on the consumer's stream when ``next()`` handed out batch ``i`` (so the ring
    slot it overwrites, used ``depth`` batches ago, is no longer being read) and runs concurrently with the work the
    consumer enqueues for batch ``i``."""

    def __init__(self, source: Iterable | Callable, device, depth: int = 2):
        self.device = torch.device(device)
        self.it: Iterator = iter(source) if not callable(source) else iter(source, None)
        self.depth = max(2, depth)
        self.stream = torch.cuda.Stream(self.device)
        self.bufs: list[torch.Tensor | None] = [None] * self.depth
        self.ready: list[torch.cuda.Event | None] = [None] * self.depth
        self.issued = 0
        self.taken = 0
        self.bytes_copied = 0
        self._issue()

    def _issue(self) -> bool:
        try:
            host = next(self.it)
        except StopIteration:
            return False
        k = self.issued % self.depth
        if self.bufs[k] is None or self.bufs[k].shape != host.shape or self.bufs[k].dtype != host.dtype:
            self.bufs[k] = torch.empty(host.shape, dtype=host.dtype, device=self.device)
        gate = torch.cuda.current_stream(self.device).record_event()
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(gate)
            self.bufs[k].copy_(host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.ready[k] = ev
        self.issued += 1
        self.bytes_copied += host.numel() * host.element_size()
        return True

    def next(self) -> torch.Tensor:
        if self.taken >= self.issued:
            raise StopIteration
        k = self.taken % self.depth
        torch.cuda.current_stream(self.device).wait_event(self.ready[k])
        out = self.bufs[k]
        self.taken += 1
        self._issue()
        return out

    __next__ = next

    def __iter__(self):
        return self
