"""Python face of the host engine (``csrc/runtime/host_engine.cpp``): CPU tensors in, asynchronous batches of
operations, a per-operation report of the device that ran it and the time it took."""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_int32, c_int64, c_uint64, c_void_p

import torch

from .. import _native

GEMM_NT, RMSNORM, GLU, ADD = range(4)
_DT = {torch.float32: 0, torch.bfloat16: 1}


class _Op(ctypes.Structure):
    _fields_ = [("kind", c_int32), ("dtype", c_int32), ("a", c_void_p), ("b", c_void_p), ("out", c_void_p),
                ("m", c_int64), ("n", c_int64), ("k", c_int64), ("lda", c_int64), ("ldb", c_int64), ("ldo", c_int64),
                ("eps", c_float), ("act", c_int32), ("seconds", c_double), ("done", c_int32), ("pad", c_int32)]


class HostEngine:
    def __init__(self, threads: int = 4):
        L = _native.lib()
        L.mesh_host_engine_create.restype = c_void_p
        L.mesh_host_engine_submit.restype = c_uint64
        L.mesh_host_engine_device.restype = ctypes.c_char_p
        self.L = L
        self.h = c_void_p(L.mesh_host_engine_create(c_int(threads)))
        self._live = {}

    @property
    def device(self) -> str:
        return self.L.mesh_host_engine_device(self.h).decode()

    @staticmethod
    def _chk(*ts):
        for t in ts:
            if t is not None and (t.is_cuda or t.dtype not in _DT or t.stride(-1) != 1):
                raise ValueError("host engine operands are CPU tensors (fp32 or bf16) with dense rows")

    def submit(self, ops: list[tuple]) -> int:
        """``ops``: tuples ``("gemm_nt", a[m,k], b[n,k], out[m,n])``, ``("rmsnorm", x[m,n], weight[n], out, eps)``,
        ``("glu", gu[m,2n], out[m,n], act)`` with ``act`` ``"silu"`` or ``"gelu_tanh"``, ``("add", a, b, out)``.
        They run in order.  Returns a ticket for :meth:`wait`."""
        arr = (_Op * len(ops))()
        keep = []
        for o, rec in zip(arr, ops):
            kind = rec[0]
            if kind == "gemm_nt":
                _, a, b, out = rec
                self._chk(a, b, out)
                o.kind, o.m, o.n, o.k = GEMM_NT, a.shape[0], b.shape[0], a.shape[1]
                o.a, o.b, o.out, o.lda, o.ldb, o.ldo = a.data_ptr(), b.data_ptr(), out.data_ptr(), a.stride(0), b.stride(0), out.stride(0)
            elif kind == "rmsnorm":
                _, a, w, out, eps = rec
                self._chk(a, w, out)
                o.kind, o.m, o.n, o.eps = RMSNORM, a.shape[0], a.shape[1], eps
                o.a, o.b, o.out, o.lda, o.ldo = a.data_ptr(), w.data_ptr(), out.data_ptr(), a.stride(0), out.stride(0)
                b = w
            elif kind == "glu":
                _, a, out, act = rec
                self._chk(a, out)
                o.kind, o.m, o.n, o.act = GLU, a.shape[0], out.shape[1], 0 if act == "silu" else 1
                o.a, o.out, o.lda, o.ldo = a.data_ptr(), out.data_ptr(), a.stride(0), out.stride(0)
                b = None
            elif kind == "add":
                _, a, b, out = rec
                self._chk(a, b, out)
                o.kind, o.m, o.n = ADD, a.shape[0], a.shape[1]
                o.a, o.b, o.out, o.lda, o.ldb, o.ldo = a.data_ptr(), b.data_ptr(), out.data_ptr(), a.stride(0), b.stride(0), out.stride(0)
            else:
                raise ValueError(kind)
            if any(t is not None and t.dtype != a.dtype for t in (b, out)):
                raise ValueError("operands of one operation share a dtype")
            o.dtype = _DT[a.dtype]
            keep.append(rec)
        ticket = int(self.L.mesh_host_engine_submit(self.h, arr, c_int(len(ops))))
        self._live[ticket] = (arr, keep)
        return ticket

    def wait(self, ticket: int, timeout_s: float = 60.0) -> list[dict]:
        """Bounded wait; returns the report ``[{op, device, seconds}]`` of the batch."""
        rc = self.L.mesh_host_engine_wait(self.h, c_uint64(ticket), c_int(int(timeout_s * 1000)))
        if rc != 0:
            raise TimeoutError(f"host engine: batch {ticket} still running after {timeout_s}s")
        arr, keep = self._live.pop(ticket)
        return [{"op": rec[0], "device": self.device, "seconds": o.seconds} for o, rec in zip(arr, keep)]

    def close(self):
        if self.h:
            for t in list(self._live):
                self.L.mesh_host_engine_wait(self.h, c_uint64(t), c_int(60000))
            self.L.mesh_host_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
