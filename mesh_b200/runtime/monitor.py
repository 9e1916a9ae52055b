"""Python face of the error monitor (``csrc/runtime/error_monitor.cu``): a host thread that reads the device status
blocks on its own stream while kernels run, spreads the abort flag after the first failure, and lets the host cancel
bounded device waits past a running kernel."""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_ulonglong, c_void_p

import torch

from .. import _native
from ..utils.status import CODES, SITES, status_block


class _Report(ctypes.Structure):
    _fields_ = [("seen_error", c_int), ("block_index", c_int), ("cuda_error", c_int), ("pad", c_int), ("polls", c_ulonglong),
                ("code", c_int), ("site", c_int), ("block", c_int), ("thread", c_int), ("expected", c_ulonglong),
                ("seen", c_ulonglong), ("aux", c_ulonglong)]


class ErrorMonitor:
    def __init__(self, device=None, blocks: list[torch.Tensor] | None = None, interval_ms: int = 5):
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.blocks = blocks or [status_block(dev)]
        arr = (c_void_p * len(self.blocks))(*[c_void_p(b.data_ptr()) for b in self.blocks])
        L = _native.lib()
        L.mesh_monitor_start.restype = c_void_p
        self.L = L
        self.h = c_void_p(L.mesh_monitor_start(c_int(dev.index or 0), arr, c_int(len(self.blocks)), c_int(interval_ms)))

    def abort(self, on: bool = True) -> None:
        """Cancel every bounded wait on the watched blocks (takes effect within a poll interval, past running kernels)."""
        self.L.mesh_monitor_abort(self.h, c_int(int(on)))

    def report(self) -> dict:
        r = _Report()
        self.L.mesh_monitor_report(self.h, ctypes.byref(r))
        return {"seen_error": bool(r.seen_error), "polls": int(r.polls), "cuda_error": r.cuda_error, "block_index": r.block_index,
                "code": CODES.get(r.code, str(r.code)), "site": SITES.get(r.site, str(r.site)), "block": r.block, "thread": r.thread,
                "expected": int(r.expected), "seen": int(r.seen)}

    def clear(self) -> None:
        self.L.mesh_monitor_clear(self.h)

    def stop(self) -> None:
        if self.h:
            self.L.mesh_monitor_stop(self.h)
            self.h = None

    def __del__(self):
        try:
            self.stop()
        except Exception:
            pass
