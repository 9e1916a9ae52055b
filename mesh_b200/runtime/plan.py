"""Persistent plans: plan once, start many.

The reference plans a program once (``mesh_plan``) and starts it many times (``mesh_transfers_start``):
executions are software-pipelined over ``copies`` buffers — execution *t* uses copy *t mod copies* — a plan
carries the membership view it was built for and is refused with ``ESTALE`` once the view has moved, and
host code can publish / wait on plan words with a no-progress bound (rdma/mesh-call.h:95-106,
rdma/mesh-dataflow.c:287-317, rdma/mesh-collective.c:17-90, :390).  Here a plan is a workspace layout
(lifetime-coloured by the native planner, repeated per copy) plus a CUDA graph per copy; ``start`` is a
graph launch.
"""
from __future__ import annotations

import ctypes
import json
import time
from ctypes import c_char_p, c_double, c_int, c_int64, c_uint64

import torch

from .. import _native
from ..config import capacity
from .rendezvous import ECANCELED, ETIMEDOUT, MeshStale

ALGOS = ["one_shot", "two_shot", "nvls", "copy_engine"]


def choose_allreduce(nbytes: int, world: int, nvls: bool = False, alpha_us: float = 2.5) -> tuple[str, float]:
    """Closed-form alpha + n*beta choice (no LP is needed for routing on a uniform fabric)."""
    L = _native.lib()
    est = c_double(0)
    a = L.mesh_plan_choose_allreduce(c_uint64(nbytes), c_int(world), c_double(alpha_us),
                                     c_double(capacity()["nvlink_gbs_per_dir"]), c_int(int(nvls)), ctypes.byref(est))
    return ALGOS[a], est.value


def layout(buffers: list[tuple[int, int, int]], copies: int = 1, align: int = 256) -> tuple[list[list[int]], int]:
    """``buffers``: ``(first step, last step, bytes)``.  Returns ``(offsets[copy][buffer], bytes per copy)``."""
    n = len(buffers)
    out = (c_int64 * max(1, n * copies))()
    L = _native.lib()
    L.mesh_plan_layout.restype = c_int64
    one = L.mesh_plan_layout(c_int(n), (c_int * max(n, 1))(*[b[0] for b in buffers]), (c_int * max(n, 1))(*[b[1] for b in buffers]),
                             (c_int64 * max(n, 1))(*[b[2] for b in buffers]), c_int64(align), c_int(copies), out)
    return [[out[c * n + i] for i in range(n)] for c in range(copies)], int(one)


VERBS = {"all_reduce": 0, "all_gather": 1, "reduce_scatter": 2, "all_to_all": 3}


class _TransferIn(ctypes.Structure):
    _fields_ = [("bytes", c_int64), ("axis", ctypes.c_int32), ("verb", ctypes.c_int32), ("at", ctypes.c_int32),
                ("read", ctypes.c_int32), ("groupable", ctypes.c_int32), ("pad", ctypes.c_int32)]


class _TransferOut(ctypes.Structure):
    _fields_ = [("demand", ctypes.c_int32), ("algo", ctypes.c_int32), ("pieces", ctypes.c_int32), ("order", ctypes.c_int32),
                ("start_us", c_double), ("end_us", c_double), ("exposed_us", c_double)]


def plan_transfers(transfers: list[dict], worlds: list[int], *, step_us: float = 10.0, alpha_us: float | None = None,
                   nvls: bool = False, bucket_bytes: int = 32 << 20, staging_bytes: int = 64 << 20) -> tuple[list[dict], dict]:
    """The native planner on a step's declared transfers.  ``transfers``: dicts with ``bytes, axis, verb, at, read`` and
    optionally ``groupable`` (a reduction that may travel with others: nothing reads it before ``read``); ``worlds``:
    ranks per axis; ``step_us``: time of one plan step in the cost model.  Returns per transfer ``{demand, algo, pieces,
    order, start_us, end_us, exposed_us}`` and the summary ``{link_us, exposed_us, makespan_us, demands}``: transfers of
    one axis grouped into demands (flat messages up to ``bucket_bytes``), an algorithm and a piece count per demand, the
    demands ordered earliest deadline first on the axis's links, and how long each reader waits."""
    n = len(transfers)
    cin = (_TransferIn * max(1, n))()
    for i, t in enumerate(transfers):
        cin[i].bytes, cin[i].axis, cin[i].verb = int(t["bytes"]), int(t.get("axis", 0)), VERBS.get(t.get("verb", "point"), 4)
        cin[i].at, cin[i].read, cin[i].groupable = int(t["at"]), int(t["read"]), int(bool(t.get("groupable", False)))
    cout = (_TransferOut * max(1, n))()
    summary = (c_double * 4)()
    cap = capacity()
    alpha = float(cap.get("collective_alpha_us", 5.0)) if alpha_us is None else alpha_us
    rc = _native.lib().mesh_plan_transfers(c_int(n), cin, c_int(len(worlds)), (c_int * max(1, len(worlds)))(*worlds),
                                           c_double(step_us), c_double(alpha), c_double(cap["nvlink_gbs_per_dir"]),
                                           c_int(int(nvls)), c_int64(bucket_bytes), c_int64(staging_bytes), cout, summary)
    if rc != 0:
        raise ValueError("plan_transfers: a transfer names an axis that does not exist, a reader before its transfer or a negative size")
    out = [{"demand": cout[i].demand, "algo": ALGOS[cout[i].algo], "pieces": cout[i].pieces, "order": cout[i].order,
            "start_us": cout[i].start_us, "end_us": cout[i].end_us, "exposed_us": cout[i].exposed_us} for i in range(n)]
    return out, {"link_us": summary[0], "exposed_us": summary[1], "makespan_us": summary[2], "demands": int(summary[3])}


def plan_pipeline(durations: list[float], resources: list[int], edges: list[tuple[int, int, int]]) -> dict:
    """The steady state of a plan started again and again (the native planner's modulo scheduler).  ``durations[i]`` and
    ``resources[i]``: time and resource (compute stream, the links of an axis, ...) of task ``i`` of one execution;
    ``edges``: ``(earlier, later, lag)`` - ``later`` of execution ``t + lag`` follows ``earlier`` of execution ``t``.
    Returns ``{period, latency, copies, resource_bound, recurrence_bound, starts}``: how often an execution can start,
    how long one takes under that schedule, how many are alive at once (the sets of buffers needed), the two lower
    bounds on the period, and every task's start within its execution."""
    n, m = len(durations), len(edges)
    if len(resources) != n:
        raise ValueError("plan_pipeline: one resource per task")
    n_res = (max(resources) + 1) if resources else 1
    starts = (c_double * max(1, n))()
    summary = (c_double * 5)()
    arr = lambda t, vals: (t * max(1, len(vals)))(*vals)       # noqa: E731
    L = _native.lib()
    rc = L.mesh_plan_pipeline(c_int(n), arr(c_double, [float(d) for d in durations]), arr(c_int, [int(r) for r in resources]),
                              c_int(n_res), c_int(m), arr(c_int, [e[0] for e in edges]), arr(c_int, [e[1] for e in edges]),
                              arr(c_int, [e[2] for e in edges]), starts, summary)
    if rc == -1:
        raise ValueError("plan_pipeline: bad input (an unknown task, a negative time or lag, or a dependence cycle within one execution)")
    if rc != 0:
        raise RuntimeError("plan_pipeline: no period found")
    return {"period": summary[0], "latency": summary[1], "copies": int(summary[2]), "resource_bound": summary[3],
            "recurrence_bound": summary[4], "starts": [starts[i] for i in range(n)]}


class Plan:
    """A captured step with ``copies`` workspaces; ``start()`` launches execution ``t`` on copy ``t % copies``."""

    def __init__(self, rdv=None, copies: int = 2, horizon: int | None = None):
        self.rdv = rdv
        self.epoch = rdv.epoch if rdv is not None else 0
        self.copies = copies
        self.horizon = horizon or copies
        self.graphs: list = [None] * copies
        self.executions = 0
        self.completions: list = []
        self.retired = False

    def capture(self, copy: int, fn) -> None:
        """Record ``fn()`` (which must only enqueue work on the current stream) as the body of ``copy``."""
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            fn()                                  # warm-up outside capture
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        # thread_local: the runtime's own service threads (status monitor, channel proxy) make CUDA calls on their own
        # streams; with the default, process-wide mode any such call during the capture invalidates it
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            fn()
        self.graphs[copy] = g

    def start(self, executions: int = 1) -> int:
        """Enqueue ``executions`` runs.  Raises ``MeshStale`` when the membership view moved since planning;
        waits (bounded) when more than ``horizon`` executions would be in flight."""
        if self.retired:
            raise RuntimeError("plan was retired")
        if self.rdv is not None:
            self.rdv.check_epoch(self.epoch)
        for _ in range(executions):
            copy = self.executions % self.copies
            if len(self.completions) >= self.horizon:
                ev = self.completions.pop(0)
                ev.synchronize()
            if self.graphs[copy] is None:
                raise RuntimeError(f"copy {copy} was never captured")
            self.graphs[copy].replay()
            ev = torch.cuda.Event()
            ev.record()
            self.completions.append(ev)
            self.executions += 1
        return self.executions

    def ended(self, execution: int) -> bool:
        done = self.executions - len([e for e in self.completions if not e.query()])
        return execution < done

    def retire(self) -> None:
        for ev in self.completions:
            ev.synchronize()
        self.completions.clear()
        self.graphs = [None] * self.copies
        self.retired = True


class HostWord:
    """A pinned host word that kernels and the host both see: publish / arrived / wait with a no-progress bound
    (``mesh_host_publish`` / ``mesh_host_arrived`` / ``mesh_host_wait``, rdma/mesh-collective.c:17-90)."""

    def __init__(self):
        # [0] what has been supplied (arrivals), [1] cancellation, [2] what has been sent (the sender may reuse its buffer)
        self.t = torch.zeros(3, dtype=torch.int64).pin_memory() if torch.cuda.is_available() else torch.zeros(3, dtype=torch.int64)

    def publish(self, value: int) -> None:
        if value > int(self.t[0]):                      # monotonic: never written to an earlier value
            self.t[0] = value

    def cancel(self) -> None:
        self.t[1] = 1

    def arrived(self, value: int) -> bool:
        return int(self.t[0]) >= value

    def mark_sent(self, value: int) -> None:
        if value > int(self.t[2]):
            self.t[2] = value

    def sent(self, value: int) -> bool:
        """Has everything up to ``value`` left this rank (``mesh_host_sent``): its source buffers may be rewritten."""
        return int(self.t[2]) >= value

    # ---- the same word seen from a CUDA stream (no kernel involved: stream memory operations)
    def _stream_words(self) -> torch.Tensor:
        """32-bit mirrors for the stream operations: [0] raised by the host for streams to wait on, [1] written by
        streams for the host to read.  Pinned, so both sides see them."""
        w = getattr(self, "_w32", None)
        if w is None:
            w = self._w32 = torch.zeros(2, dtype=torch.int32).pin_memory()
        return w

    def publish_to_streams(self, value: int) -> None:
        """``publish`` that streams blocked in :meth:`stream_wait` also see (monotonic)."""
        self.publish(value)
        w = self._stream_words()
        if value > int(w[0]):
            w[0] = value

    def stream_wait(self, value: int, stream=None) -> None:
        """Everything queued on ``stream`` (default: the current one) after this call starts only once the word has
        been published to at least ``value`` - the device-side counterpart of :meth:`wait`, without a polling kernel
        (``cuStreamWaitValue32``).  The host must publish in finite time: a stream wait has no timeout of its own."""
        from ctypes import c_uint32, c_void_p
        s = (stream or torch.cuda.current_stream()).cuda_stream
        w = self._stream_words()
        rc = _native.lib().mesh_stream_wait_value(c_void_p(s), c_void_p(w.data_ptr()), c_uint32(value & 0xFFFFFFFF))
        _native.check(rc, "mesh_stream_wait_value")

    def stream_mark_sent(self, value: int, stream=None) -> None:
        """The stream records ``value`` once everything queued before this call has finished; :meth:`stream_sent`
        reads it (``cuStreamWriteValue32``): the host learns that a buffer has left without synchronising."""
        from ctypes import c_uint32, c_void_p
        s = (stream or torch.cuda.current_stream()).cuda_stream
        w = self._stream_words()
        rc = _native.lib().mesh_stream_write_value(c_void_p(s), c_void_p(w.data_ptr() + 4), c_uint32(value & 0xFFFFFFFF))
        _native.check(rc, "mesh_stream_write_value")

    def stream_sent(self, value: int) -> bool:
        return int(self._stream_words()[1]) >= value

    def wait(self, value: int, timeout_s: float = 5.0) -> int:
        """0 when reached, ``ECANCELED`` when cancelled, ``ETIMEDOUT`` after ``timeout_s`` without progress."""
        last, t_last = int(self.t[0]), time.monotonic()
        while True:
            cur = int(self.t[0])
            if cur >= value:
                return 0
            if int(self.t[1]):
                return ECANCELED
            if cur != last:
                last, t_last = cur, time.monotonic()
            elif time.monotonic() - t_last > timeout_s:
                return ETIMEDOUT
            time.sleep(0.0005)


def save(path: str, epoch: int, words: list[int]) -> None:
    arr = (c_uint64 * max(1, len(words)))(*words)
    rc = _native.lib().mesh_plan_save(c_char_p(str(path).encode()), c_uint64(epoch), arr, c_uint64(len(words)))
    if rc != 0:
        raise OSError(f"mesh_plan_save({path}) failed: {rc}")


def load(path: str, cap: int = 1 << 20) -> tuple[int, list[int]]:
    arr = (c_uint64 * cap)()
    ep = c_uint64(0)
    L = _native.lib()
    L.mesh_plan_load.restype = c_int64
    n = L.mesh_plan_load(c_char_p(str(path).encode()), ctypes.byref(ep), arr, c_uint64(cap))
    if n < 0:
        raise OSError({-1: "cannot open", -2: "bad header", -3: "checksum mismatch", -4: "too large"}.get(n, str(n)) + f": {path}")
    return int(ep.value), list(arr[:n])
