"""Communicator: the collective verbs on CUDA tensors, run by this package's own kernels.

One ``Communicator`` per (set of ranks, symmetric heap).  It owns two staging buffers (alternated
call by call — the reference's ``copies`` buffers, rdma/mesh-flow.c:7-12), their arrival counters
(monotonic, never reset) and the point-to-point slots.  Every verb is explicit — nothing is
inferred from the number of peers (design/collective-verbs.md:7-35) — and the v-variants carry
per-rank counts so unequal shards move at their own sizes
(design/unequal-shards-change-request.md:73-476).

All ranks must issue the same sequence of collectives with consistent sizes, as with any
``torch.distributed`` backend; the expected counter values are derived from that sequence, so no
sequence numbers travel between ranks.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_uint32, c_uint64, c_void_p

import torch

from .. import _native
from ..config import config
from ..runtime.heap import SymmetricHeap
from ..utils.status import status_block

MAX_RANKS = 8
HEADER = 1024
F32, BF16, F16, I32, I64, U8, F64 = range(7)
SUM, MAX, MIN, PROD, AVG = range(5)

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16, torch.int32: I32, torch.int64: I64,
       torch.uint8: U8, torch.bool: U8, torch.float64: F64}
_OPS = {"sum": SUM, "max": MAX, "min": MIN, "prod": PROD, "product": PROD, "avg": AVG}


class _CommArgs(ctypes.Structure):
    _fields_ = [("rank", c_int), ("world", c_int), ("staging", c_void_p * MAX_RANKS), ("arrived", c_void_p * MAX_RANKS),
                ("expect_a", c_uint32), ("expect_b", c_uint32), ("add", c_uint32), ("staging_bytes", c_uint64),
                ("status", c_void_p), ("nblocks", c_int)]


class _XferChan(ctypes.Structure):
    _fields_ = [("slot", c_void_p), ("ready", c_void_p), ("ack", c_void_p), ("ready_base", c_uint32), ("ack_base", c_uint32)]


class _XferArgs(ctypes.Structure):
    _fields_ = [("n_send", c_int), ("has_recv", c_int), ("nb", c_int), ("depth", c_int), ("send", _XferChan * MAX_RANKS),
                ("recv", _XferChan), ("inp", c_void_p), ("out", c_void_p), ("send_bytes", c_uint64), ("recv_bytes", c_uint64),
                ("piece", c_uint64), ("status", c_void_p)]


P2P_DEPTH = 4


def _op_code(op) -> int:
    if isinstance(op, int):
        return op
    name = str(op).lower().split(".")[-1]
    name = {"redoptype.sum": "sum"}.get(name, name)
    if name not in _OPS:
        raise ValueError(f"unsupported reduce op {op!r}")
    return _OPS[name]


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class Communicator:
    def __init__(self, heap: SymmetricHeap, staging_bytes: int = 64 << 20, p2p_slot_bytes: int = 32 << 20):
        self.heap = heap
        self.rank, self.world = heap.rank, heap.world
        if self.world > MAX_RANKS:
            raise ValueError(f"mesh communicator supports up to {MAX_RANKS} ranks per node")
        self.staging_bytes = staging_bytes
        self._staging = [heap.alloc((HEADER + staging_bytes,), torch.uint8) for _ in range(2)]
        self._arrived = [heap.alloc_signals(2 * self.world) for _ in range(2)]
        self._expect = [[0, 0], [0, 0]]
        self._turn = 0
        self.p2p_slot_bytes = p2p_slot_bytes // (P2P_DEPTH * 16) * (P2P_DEPTH * 16)
        self._slots = heap.alloc((self.world, self.p2p_slot_bytes), torch.uint8)   # ring[dst] on the sender
        self._ready = heap.alloc_signals(self.world)                          # ready[src] on the receiver
        self._ack = heap.alloc_signals(self.world)                            # ack[dst] on the sender
        self._sent = [0] * self.world          # block arrivals raised so far on the channel to each destination
        self._rcvd = [0] * self.world          # ... and on the channel from each source
        self.L = _native.lib()
        self.max_blocks = self.L.mesh_coll_max_blocks()
        self.one_shot_max = self._one_shot_threshold()
        self._svc = None
        try:
            from .context import current_or_none
            from ..runtime import service
            ctx = current_or_none()
            if ctx is not None and ctx.service:
                self._svc = service
        except Exception:
            self._svc = None
        self.use_nvls = bool(config().nvls and getattr(heap, "mc_ptr", 0))
        self.calls = 0

    # ------------------------------------------------------------------ plumbing
    def _one_shot_threshold(self) -> int:
        """Largest message that goes one-shot.  ``MESH_ONE_SHOT_MAX`` when set; otherwise the planner's latency +
        bytes / bandwidth model decides (one-shot moves ``(world - 1) x n`` bytes into every rank in one round,
        two-shot ``2 (world - 1) / world x n`` in two): the threshold is where its choice changes."""
        import os
        if os.environ.get("MESH_ONE_SHOT_MAX") or self.world == 1:
            return config().one_shot_max_bytes
        try:
            from ..config import capacity
            from ..runtime.plan import choose_allreduce as _choose
            alpha = float(capacity().get("collective_alpha_us", 5.0))      # measured launch-to-first-byte latency
            choose_allreduce = lambda n, w: _choose(n, w, False, alpha)
            lo, hi = 1 << 10, 64 << 20
            if choose_allreduce(lo, self.world)[0] != "one_shot":
                return lo
            while hi - lo > (4 << 10):
                mid = (lo + hi) // 2
                if choose_allreduce(mid, self.world)[0] == "one_shot":
                    lo = mid
                else:
                    hi = mid
            return min(lo, self.staging_bytes)
        except Exception:
            return config().one_shot_max_bytes

    def _blocks(self, nbytes: int) -> int:
        # one 16-byte vector per thread (512 threads) until every SM has a block
        return max(1, min(self.max_blocks, (nbytes + (8 << 10) - 1) // (8 << 10)))

    def _args(self, nblocks: int, two_step: bool = False) -> _CommArgs:
        par = self._turn & 1
        self._turn += 1
        self.calls += 1
        self._expect[par][0] += nblocks
        if two_step:
            self._expect[par][1] += nblocks
        a = _CommArgs()
        a.rank, a.world = self.rank, self.world
        for r in range(self.world):
            a.staging[r] = self._staging[par].ptr(r)
            a.arrived[r] = self._arrived[par].ptr(r)
        a.expect_a, a.expect_b = self._expect[par][0], self._expect[par][1]
        a.add = 1
        a.staging_bytes = self.staging_bytes
        a.status = status_block(self.heap.device).data_ptr()
        a.nblocks = nblocks
        if self._svc is not None:
            self._svc.count("collectives", 1)
        return a

    def _bytes_out(self, per_peer: int) -> None:
        """Stats block of the runtime service: bytes this rank's links carry to each peer for one collective."""
        if self._svc is not None and per_peer:
            for peer in range(self.world):
                if peer != self.rank:
                    self._svc.count("bytes", per_peer, peer)

    @staticmethod
    def _check(t: torch.Tensor, name: str) -> None:
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CUDA tensor")

    def _dtype(self, t: torch.Tensor) -> int:
        if t.dtype not in _DT:
            raise TypeError(f"mesh collectives do not reduce {t.dtype}")
        return _DT[t.dtype]

    # ------------------------------------------------------------------ reductions
    def all_reduce(self, t: torch.Tensor, op="sum", out: torch.Tensor | None = None) -> torch.Tensor:
        """In place unless ``out`` is given.  One-shot below ``one_shot_max_bytes``, two-shot above;
        messages larger than the staging buffer go in pieces."""
        self._check(t, "tensor")
        out = t if out is None else out
        dt, opc = self._dtype(t), _op_code(op)
        es = t.element_size()
        n = t.numel()
        flat_in, flat_out = t.view(-1), out.view(-1)
        cap_two = (self.staging_bytes // 2 // 16 * 16) // es
        pos = 0
        while pos < n or n == 0:
            cnt = min(n - pos, cap_two)
            nbytes = cnt * es
            two = nbytes > self.one_shot_max and self.world > 1
            nb = self._blocks(nbytes)
            mc = self._staging[self._turn & 1].mc_ptr if (self.use_nvls and two and opc == SUM and dt in (F32, BF16, F16)) else 0
            if mc:
                # in-switch reduction: the heap has a multicast mapping (MESH_NVLS=1)
                a = self._args(nb, two_step=True)
                rc = self.L.mesh_coll_allreduce_mc(ctypes.byref(a), c_void_p(mc), c_void_p(flat_in[pos:].data_ptr()),
                                                   c_void_p(flat_out[pos:].data_ptr()), c_uint64(cnt), c_int(dt), _stream())
                _native.check(rc, "mesh_coll_allreduce_mc")
                _native.count_launch()
                pos += cnt
                continue
            self._bytes_out(nbytes if not two else 2 * nbytes // self.world)
            a = self._args(nb, two_step=two)
            rc = self.L.mesh_coll_allreduce(ctypes.byref(a), c_void_p(flat_in[pos:].data_ptr() if n else 0),
                                            c_void_p(flat_out[pos:].data_ptr() if n else 0), c_uint64(cnt), c_int(dt),
                                            c_int(opc), c_int(int(two)), _stream())
            _native.check(rc, "mesh_coll_allreduce")
            _native.count_launch()
            pos += cnt
            if n == 0:
                break
        return out

    def reduce_scatter(self, out: torch.Tensor, inp: torch.Tensor, op="sum", counts: list[int] | None = None):
        """``out`` = this rank's segment of the elementwise reduction of every rank's ``inp``.
        ``counts[r]``: elements owned by rank r (default: equal)."""
        self._check(out, "out"); self._check(inp, "inp")
        if counts is None:
            counts = [inp.numel() // self.world] * self.world
        if sum(counts) != inp.numel() or counts[self.rank] != out.numel():
            raise ValueError("reduce_scatter: counts do not match the tensors")
        if inp.numel() * inp.element_size() > self.staging_bytes:
            return self._reduce_scatter_pieces(out, inp, op, counts)
        arr = (c_uint64 * self.world)(*counts)
        self._bytes_out(inp.numel() * inp.element_size() // self.world)
        a = self._args(self._blocks(inp.numel() * inp.element_size()))
        rc = self.L.mesh_coll_reduce_scatter(ctypes.byref(a), c_void_p(inp.data_ptr()), c_void_p(out.data_ptr()), arr,
                                             c_int(self._dtype(inp)), c_int(_op_code(op)), _stream())
        _native.check(rc, "mesh_coll_reduce_scatter")
        _native.count_launch()
        return out

    def _reduce_scatter_pieces(self, out, inp, op, counts):
        # Too large for one staging buffer: cut every rank's segment into the same number of pieces.
        es = inp.element_size()
        pieces = (inp.numel() * es + self.staging_bytes - 1) // self.staging_bytes
        displs = [0]
        for c in counts:
            displs.append(displs[-1] + c)
        flat_in, flat_out = inp.view(-1), out.view(-1)
        for p in range(pieces):
            sub_counts, parts = [], []
            for r, c in enumerate(counts):
                lo, hi = c * p // pieces, c * (p + 1) // pieces
                sub_counts.append(hi - lo)
                parts.append(flat_in[displs[r] + lo: displs[r] + hi])
            mine_lo = counts[self.rank] * p // pieces
            self.reduce_scatter(flat_out[mine_lo: mine_lo + sub_counts[self.rank]], torch.cat(parts), op, sub_counts)
        return out

    def reduce(self, t: torch.Tensor, root: int, op="sum") -> torch.Tensor:
        self._check(t, "tensor")
        es, n = t.element_size(), t.numel()
        cap = self.staging_bytes // es
        flat = t.view(-1)
        pos = 0
        while pos < n:
            cnt = min(n - pos, cap)
            a = self._args(self._blocks(cnt * es))
            rc = self.L.mesh_coll_reduce(ctypes.byref(a), c_void_p(flat[pos:].data_ptr()), c_void_p(flat[pos:].data_ptr()),
                                         c_uint64(cnt), c_int(self._dtype(t)), c_int(_op_code(op)), c_int(root), _stream())
            _native.check(rc, "mesh_coll_reduce")
            _native.count_launch()
            pos += cnt
        return t

    # ------------------------------------------------------------------ data movement
    def all_gather(self, out: torch.Tensor, inp: torch.Tensor, counts: list[int] | None = None):
        """``out`` = concatenation of every rank's ``inp``; ``counts[r]`` elements from rank r."""
        self._check(out, "out"); self._check(inp, "inp")
        es = inp.element_size()
        if counts is None:
            counts = [inp.numel()] * self.world
        if counts[self.rank] != inp.numel() or sum(counts) != out.numel():
            raise ValueError("all_gather: counts do not match the tensors")
        displs = [0]
        for c in counts:
            displs.append(displs[-1] + c)
        cap = self.staging_bytes // es
        pieces = max(1, (max(counts) + cap - 1) // cap)
        flat_in, flat_out = inp.view(-1), out.view(-1)
        self._bytes_out(inp.numel() * es)
        for p in range(pieces):
            lo = [c * p // pieces for c in counts]
            hi = [c * (p + 1) // pieces for c in counts]
            cb = (c_uint64 * self.world)(*[(h - l) * es for l, h in zip(lo, hi)])
            db = (c_uint64 * self.world)(*[(displs[r] + lo[r]) * es for r in range(self.world)])
            a = self._args(self._blocks(max(h - l for l, h in zip(lo, hi)) * es))
            src = flat_in[lo[self.rank]:]
            rc = self.L.mesh_coll_allgatherv(ctypes.byref(a), c_void_p(src.data_ptr() if src.numel() else 0),
                                             c_void_p(flat_out.data_ptr()), cb, db, _stream())
            _native.check(rc, "mesh_coll_allgatherv")
            _native.count_launch()
        return out

    def all_to_all(self, out: torch.Tensor, inp: torch.Tensor, out_splits: list[int] | None = None,
                   in_splits: list[int] | None = None):
        """MPI_Alltoallv over dim 0: ``in_splits[j]`` rows go to rank j, ``out_splits[j]`` rows come from it."""
        self._check(out, "out"); self._check(inp, "inp")
        W = self.world
        row_elems = 1
        for d in inp.shape[1:]:
            row_elems *= d
        row_bytes = row_elems * inp.element_size()
        if in_splits is None:
            in_splits = [inp.shape[0] // W] * W
        if out_splits is None:
            out_splits = [out.shape[0] // W] * W
        soff, roff = [0], [0]
        for j in range(W):
            soff.append(soff[-1] + in_splits[j] * row_bytes)
            roff.append(roff[-1] + out_splits[j] * row_bytes)
        if soff[-1] > self.staging_bytes:
            raise ValueError(f"all_to_all: {soff[-1]} bytes exceed the staging buffer ({self.staging_bytes}); "
                             "raise staging_bytes or split the call")
        self._bytes_out(soff[-1] // max(1, W))
        a = self._args(32)
        rc = self.L.mesh_coll_alltoallv(ctypes.byref(a), c_void_p(inp.data_ptr()), c_void_p(out.data_ptr()),
                                        (c_uint64 * (W + 1))(*soff), (c_uint64 * (W + 1))(*roff), _stream())
        _native.check(rc, "mesh_coll_alltoallv")
        _native.count_launch()
        return out

    def broadcast(self, t: torch.Tensor, root: int) -> torch.Tensor:
        self._check(t, "tensor")
        flat = t.view(-1).view(torch.uint8) if t.dtype != torch.bool else t.view(-1).view(torch.uint8)
        n = flat.numel()
        pos = 0
        while pos < n:
            cnt = min(n - pos, self.staging_bytes)
            a = self._args(self._blocks(cnt))
            rc = self.L.mesh_coll_broadcast(ctypes.byref(a), c_void_p(flat[pos:].data_ptr()), c_uint64(cnt), c_int(root),
                                            _stream())
            _native.check(rc, "mesh_coll_broadcast")
            _native.count_launch()
            pos += cnt
        return t

    def gather(self, out: torch.Tensor | None, inp: torch.Tensor, root: int):
        """Root receives every rank's ``inp`` (equal sizes) into ``out[world, ...]``."""
        rows = inp.numel()
        flat_in = inp.reshape(1, -1)
        if self.rank == root:
            dst = out.view(self.world, -1)
            self.all_to_all(dst, flat_in.expand(1, rows).contiguous(), out_splits=[1] * self.world,
                            in_splits=[1 if j == root else 0 for j in range(self.world)])
        else:
            empty = torch.empty((0, rows), dtype=inp.dtype, device=inp.device)
            self.all_to_all(empty, flat_in.contiguous(), out_splits=[0] * self.world,
                            in_splits=[1 if j == root else 0 for j in range(self.world)])
        return out

    def scatter(self, out: torch.Tensor, inp: torch.Tensor | None, root: int):
        """Rank r receives ``inp[r]`` of the root's ``inp[world, ...]``."""
        rows = out.numel()
        dst = out.view(1, -1)
        if self.rank == root:
            src = inp.reshape(self.world, rows).contiguous()
            self.all_to_all(dst, src, out_splits=[1 if j == root else 0 for j in range(self.world)],
                            in_splits=[1] * self.world)
        else:
            src = torch.empty((0, rows), dtype=out.dtype, device=out.device)
            self.all_to_all(dst, src, out_splits=[1 if j == root else 0 for j in range(self.world)],
                            in_splits=[0] * self.world)
        return out

    def barrier(self) -> None:
        a = self._args(1)
        _native.check(self.L.mesh_coll_barrier(ctypes.byref(a), _stream()), "mesh_coll_barrier")
        _native.count_launch()

    # ------------------------------------------------------------------ point to point
    def _p2p_blocks(self, nbytes: int) -> int:
        return max(1, min(48, nbytes // (64 << 10)))

    def _exchange(self, inp, dsts: list[int], out, src: int | None) -> None:
        """One launch: ``inp`` goes to every rank of ``dsts`` and ``out`` is filled from ``src``.  Both ends of a
        channel derive the piece count and the block count from the message size, so their counters agree."""
        piece = self.p2p_slot_bytes // P2P_DEPTH
        a = _XferArgs()
        a.depth, a.piece = P2P_DEPTH, piece
        a.status = status_block(self.heap.device).data_ptr()
        sb = inp.numel() * inp.element_size() if inp is not None else 0
        rb = out.numel() * out.element_size() if out is not None else 0
        nbytes = max(sb if dsts else 0, rb if src is not None else 0)
        nb = self._p2p_blocks(nbytes)
        if dsts and src is not None and sb != rb:
            raise ValueError("exchange: this rank's send and receive sizes differ; use send and recv")
        a.nb = nb
        a.n_send = len(dsts)
        for i, d in enumerate(dsts):
            ch = a.send[i]
            ch.slot = self._slots.ptr(self.rank) + d * self.p2p_slot_bytes
            ch.ready = self._ready.ptr(d) + 4 * self.rank
            ch.ack = self._ack.ptr(self.rank) + 4 * d
            ch.ready_base = ch.ack_base = self._sent[d] & 0xFFFFFFFF
            self._sent[d] += -(-sb // piece) * nb
        a.has_recv = int(src is not None)
        if src is not None:
            ch = a.recv
            ch.slot = self._slots.ptr(src) + self.rank * self.p2p_slot_bytes
            ch.ready = self._ready.ptr(self.rank) + 4 * src
            ch.ack = self._ack.ptr(src) + 4 * self.rank
            ch.ready_base = ch.ack_base = self._rcvd[src] & 0xFFFFFFFF
            self._rcvd[src] += -(-rb // piece) * nb
        a.inp = inp.data_ptr() if (inp is not None and sb) else 0
        a.out = out.data_ptr() if (out is not None and rb) else 0
        a.send_bytes, a.recv_bytes = sb, rb
        if a.n_send == 0 and not a.has_recv:
            return
        _native.check(self.L.mesh_p2p_exchange(ctypes.byref(a), _stream()), "mesh_p2p_exchange")
        _native.count_launch()

    def send(self, t: torch.Tensor, dst: int) -> None:
        """Stage ``t`` piece by piece in this rank's ring for ``dst``, from which the receiver pulls it.  Finishes (on
        the stream) once the last piece is staged: a message no larger than the ring does not wait for the receiver."""
        self._check(t, "tensor")
        self._exchange(t.view(-1).view(torch.uint8), [dst], None, None)

    def recv(self, t: torch.Tensor, src: int) -> torch.Tensor:
        self._check(t, "tensor")
        self._exchange(None, [], t.view(-1).view(torch.uint8), src)
        return t

    def permute(self, out: torch.Tensor, inp: torch.Tensor, pairs: list[tuple[int, int]]):
        """collective-permute: for every ``(src, dst)`` pair, ``out`` on dst = ``inp`` on src
        (rdma/mesh_compile.py:1597-1613).  Sending and receiving run in the same launch, so a ring of messages of
        any size cannot have every rank waiting to send."""
        dsts = [d for s_, d in pairs if s_ == self.rank]
        srcs = [s_ for s_, d in pairs if d == self.rank]
        if len(srcs) > 1:
            raise ValueError("permute: a rank receives from at most one source")
        fin = inp.view(-1).view(torch.uint8) if dsts else None
        fout = out.view(-1).view(torch.uint8) if srcs else None
        if fin is not None and fout is not None and fin.numel() != fout.numel():
            # unequal sizes: the receive must not share a launch geometry with the sends
            self._exchange(fin, dsts, None, None)
            self._exchange(None, [], fout, srcs[0])
            return out
        self._exchange(fin, dsts, fout, srcs[0] if srcs else None)
        return out
