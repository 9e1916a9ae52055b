"""Sequence-parallel tensor-parallel gated FFN on fused compute+collective kernels.

Megatron-style split (reference placement ``megatron()``, examples/parallel.py:77-89): gate/up
weights column-parallel, down weight row-parallel, activations sharded along the token
dimension between layers.  The reference's compiler would emit an all-gather before the column
GEMM and a reduce(-scatter) after the row GEMM (compiler/mesh_compiler/placement.py:250-340,
:812-834); here each pair is ONE kernel:

  forward   1. push x shard to every rank's gathered buffer  +  [g|u] = X Wgu^T, h = act(g)*u
            2. partial y = h Wd^T, tiles stored to the owner rank  +  owner sums the partials
  backward  3. push dy shard  +  dH = dY Wd with the GLU backward in the epilogue -> [dg|du]
            4. dWd  = dY^T h
            5. partial dx = [dg|du] Wgu, scattered + reduced like (2)
            6. dWgu = [dg|du]^T X

Buffers that peers write into are double-buffered by use parity; their arrival counters only ever
increase, so no barrier or reset is needed between steps (same idea as the reference's
``copies`` buffers and monotonic words, rdma/mesh-flow.c:7-15).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from ..ops import gemm as G
from ..runtime.heap import SymmetricHeap
from ..utils.status import status_block

BM, BN = 128, 256
AG_SPLIT = 8
EPI_WARPS = 4


class _Gathered:
    """An all-gather landing zone [M, D] with per-128-row arrival counters, ``copies`` buffers used in turn.

    Two copies are enough for the exchange itself (a rank can be at most one use ahead of a peer).  The gathered
    tensor is also what the weight-gradient GEMM of the backward pass reads, so a caller that runs several forward
    passes before the matching backward passes (pipeline microbatches) asks for as many copies as passes in flight."""

    def __init__(self, heap: SymmetricHeap, M: int, D: int, copies: int = 2):
        copies = max(2, copies)
        self.copies = copies
        # parts a 128-row block is pushed in.  Measured at 8 GPUs: cutting blocks finer, so that all CTAs push to one
        # destination at a time, is slower (653 us per step against 626 us): every part ends with a system-scope
        # release that waits for the part's stores to be acknowledged across NVLink, and the parts of a CTA run one
        # after the other
        self.split = AG_SPLIT
        self.buf = [heap.alloc((M, D), torch.bfloat16) for _ in range(copies)]
        self.flags = [heap.alloc_signals(M // BM) for _ in range(copies)]
        self.uses = [0] * copies
        self.turn = 0

    def next(self):
        par = self.turn % self.copies
        self.turn += 1
        self.uses[par] += 1
        return self.buf[par], self.flags[par], self.split * self.uses[par]


class _Scattered:
    """A double-buffered reduce-scatter landing zone [world, M/world, N] with per-tile counters."""

    def __init__(self, heap: SymmetricHeap, world: int, rows: int, N: int):
        self.world = world
        # tile width the launcher would pick for the whole [world*rows, N] product
        self.tile_n = _native.lib().mesh_gemm_choose_tile_n(world * rows, N, 0)
        bn = self.tile_n
        # tile-contiguous: [src rank][m-tile][n-tile][128*bn]
        self.buf = [heap.alloc((world, rows // BM, (N + bn - 1) // bn, BM * bn), torch.bfloat16) for _ in range(2)]
        self.count = [heap.alloc_signals((rows // BM) * ((N + bn - 1) // bn)) for _ in range(2)]
        self.uses = [0, 0]
        self.turn = 0

    def next(self):
        par = self.turn & 1
        self.turn += 1
        self.uses[par] += 1
        return self.buf[par], self.count[par], self.world * EPI_WARPS * self.uses[par]


def shared_zone(heap, cls, *shape):
    """Landing zones that hold data only while one kernel pair runs (reduce-scatter partials, gathered gradients) are
    shared by every layer of the same shape on a heap: layers run one after the other, and the zones' counters are
    monotonic, so consecutive users simply continue the sequence.  (The gathered activations are not shared: the
    backward pass reads them again.)"""
    zones = heap.__dict__.setdefault("_zones", {})
    key = (cls.__name__, *shape)
    if key not in zones:
        zones[key] = cls(heap, *shape)
    return zones[key]


class FusedTPFFN:
    """Holds the symmetric workspaces of one (M, D, F) FFN shape and runs its six fused kernels.

    ``w_gate_up``: this rank's ``[2*Fl, D]`` (gate rows, then up rows); ``w_down``: ``[D, Fl]``, with ``Fl = F / world``
    or, for unequal shares of the hidden units (heterogeneous ranks, ``runtime/allocate.py``), ``ff_local``: any
    multiple of 64; the ranks' shares add up to ``F``.  The hidden width is a local dimension of every kernel here (the
    gathered and scattered dimension is the tokens'), so ranks with different shares run the same six launches and only
    differ in how long they compute.
    """

    def __init__(self, heap: SymmetricHeap, tokens: int, d_model: int, d_ff: int, act: str = "silu", in_flight: int = 1,
                 ff_local: int | None = None):
        self.heap = heap
        self.rank, self.world = heap.rank, heap.world
        self.M, self.D, self.F = tokens, d_model, d_ff
        self.act = act
        P = self.world
        if tokens % (P * BM):
            raise ValueError(f"tokens ({tokens}) must be a multiple of world*128")
        if ff_local is None:
            if d_ff % P:
                raise ValueError("d_ff must be a multiple of the world size (or pass ff_local)")
            ff_local = d_ff // P
        if ff_local % 64 or ff_local <= 0 or d_model % 64:
            raise ValueError("this rank's share of d_ff and d_model must be multiples of 64")
        self.rows = tokens // P
        self.Fl = ff_local
        self.x_full = _Gathered(heap, tokens, d_model, copies=in_flight + 1)
        self.dy_full = shared_zone(heap, _Gathered, tokens, d_model)
        self.y_recv = shared_zone(heap, _Scattered, P, self.rows, d_model)
        self.dx_recv = self.y_recv          # forward and backward never overlap within a rank's stream
        self._saved = None
        # Row-block completion counters of the two matrices that one launch of a pass writes and the next launches
        # read while the writer's last tiles are still running (h in the forward pass, [dg|du] in the backward pass).
        self.chain = G.chaining()
        self.done_h = G.Done(heap.device, tokens // BM)
        self.done_dgu = G.Done(heap.device, tokens // BM)
        self.bwd_tile_n = G.tile_n_for(tokens, self.Fl)

    # ---------------------------------------------------------------- kernels
    def _args(self, dev) -> _native.GemmArgs:
        g = _native.GemmArgs()
        g.status = status_block(dev).data_ptr()
        g.rank, g.world = self.rank, self.world
        return g

    def _gather_args(self, g, zone: _Gathered, src: torch.Tensor):
        buf, flags, expect = zone.next()
        g.A, g.lda, g.a_rows = buf.ptr(), self.D, self.M
        g.a_ready, g.a_ready_value, g.a_ready_rows = flags.ptr(), expect, BM
        g.m_rotate = self.rank * (self.rows // BM)
        g.ag_src, g.ag_rows_per_rank, g.ag_ld = src.data_ptr(), self.rows, self.D
        g.ag_split = zone.split
        for r in range(self.world):
            g.ag_dst[r] = buf.ptr(r)
            g.ag_flags[r] = flags.ptr(r)
        self._gathered_ready = (flags.ptr(), expect, BM)
        return buf

    def _scatter_args(self, g, zone: _Scattered, out: torch.Tensor):
        buf, count, expect = zone.next()
        g.epi = G.EPI_SCATTER
        g.tile_n = zone.tile_n
        for r in range(self.world):
            g.rs_recv[r] = buf.ptr(r)
            g.rs_count[r] = count.ptr(r)
        g.rs_expect, g.rs_out, g.rs_rows_per_rank = expect, out.data_ptr(), self.rows
        g.m_rotate = ((self.rank + 1) % self.world) * (self.rows // BM)   # own rows last

    def forward(self, x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, save: bool = True):
        """x: this rank's ``[M/world, D]`` token shard -> y shard ``[M/world, D]``."""
        dev = x.device
        M, D, Fl = self.M, self.D, self.Fl
        h = torch.empty((M, Fl), dtype=torch.bfloat16, device=dev)
        gu = torch.empty((M, 2 * Fl), dtype=torch.bfloat16, device=dev) if save else None
        # (1) all-gather(x) -> GLU GEMM
        g = self._args(dev)
        xbuf = self._gather_args(g, self.x_full, x)
        g.B, g.ldb, g.b_rows, g.b_up_rows = w_gate_up.data_ptr(), w_gate_up.stride(0), 2 * Fl, Fl
        g.M, g.N, g.K = M, Fl, D
        g.epi, g.act = G.EPI_GLU_FWD, G.ACT[self.act]
        g.D, g.ldd, g.d_cols = h.data_ptr(), Fl, Fl
        if save:
            g.D2, g.ldd2, g.d2_cols, g.d_up_cols = gu.data_ptr(), 2 * Fl, 2 * Fl, Fl
        if self.chain:
            G.chain(g, d_done=self.done_h, trigger=True)
        G._launch(g)
        # (2) down GEMM -> reduce-scatter; starts during the last wave of (1) and reads h row block by row block
        y = torch.empty((self.rows, D), dtype=torch.bfloat16, device=dev)
        g = self._args(dev)
        g.A, g.lda, g.a_rows = h.data_ptr(), Fl, M
        g.B, g.ldb, g.b_rows = w_down.data_ptr(), w_down.stride(0), D
        g.M, g.N, g.K = M, D, Fl
        self._scatter_args(g, self.y_recv, y)
        if self.chain:
            G.chain(g, a_ready=(self.done_h.ptr(), self.done_h.produce((Fl + 127) // 128), BM), dependent=True)
        G._launch(g)
        if save:
            self._saved = (xbuf, h, gu, w_gate_up, w_down)
        return y

    def backward(self, dy: torch.Tensor):
        """dy: ``[M/world, D]`` -> ``(dx shard, dW_gate_up, dW_down)``."""
        xbuf, h, gu, w_gate_up, w_down = self._saved
        dev = dy.device
        M, D, Fl = self.M, self.D, self.Fl
        dy = dy.contiguous()
        # (3) all-gather(dy) -> dH GEMM with GLU backward epilogue
        dgu = torch.empty((M, 2 * Fl), dtype=torch.bfloat16, device=dev)
        g = self._args(dev)
        dybuf = self._gather_args(g, self.dy_full, dy)
        g.B, g.ldb, g.b_mn = w_down.data_ptr(), w_down.stride(0), 1
        g.M, g.N, g.K = M, Fl, D
        g.epi, g.act = G.EPI_GLU_BWD, G.ACT[self.act]
        g.aux, g.ld_aux, g.d_up_cols = gu.data_ptr(), 2 * Fl, Fl
        g.D, g.ldd, g.d_cols = dgu.data_ptr(), 2 * Fl, 2 * Fl
        g.tile_n = self.bwd_tile_n
        dy_ready = self._gathered_ready          # dY row blocks in this rank's gathered buffer (arrival counters)
        if not self.chain:
            G._launch(g)
            dw_down = G.gemm(dybuf.local, h, a_mn=True, b_mn=True)
            dx = torch.empty((self.rows, D), dtype=torch.bfloat16, device=dev)
            g = self._args(dev)
            g.A, g.lda, g.a_rows = dgu.data_ptr(), 2 * Fl, M
            g.B, g.ldb, g.b_mn = w_gate_up.data_ptr(), w_gate_up.stride(0), 1
            g.M, g.N, g.K = M, D, 2 * Fl
            self._scatter_args(g, self.dx_recv, dx)
            G._launch(g)
            dw_gate_up = G.gemm(dgu, xbuf.local, a_mn=True, b_mn=True)
            return dx, dw_gate_up, dw_down
        # The four launches overlap: each starts during the last wave of the one before it and waits, row block by row
        # block, for what it reads of (3)'s outputs.  dx goes first: the layer below waits for it.
        G.chain(g, d_done=self.done_dgu, trigger=True)
        G._launch(g)
        dgu_ready = (self.done_dgu.ptr(), self.done_dgu.produce((Fl + self.bwd_tile_n - 1) // self.bwd_tile_n), BM)
        # (5) dx partial = [dg|du] Wgu -> reduce-scatter
        dx = torch.empty((self.rows, D), dtype=torch.bfloat16, device=dev)
        g = self._args(dev)
        g.A, g.lda, g.a_rows = dgu.data_ptr(), 2 * Fl, M
        g.B, g.ldb, g.b_mn = w_gate_up.data_ptr(), w_gate_up.stride(0), 1
        g.M, g.N, g.K = M, D, 2 * Fl
        self._scatter_args(g, self.dx_recv, dx)
        G.chain(g, a_ready=dgu_ready, dependent=True, trigger=True)
        G._launch(g)
        # (4) dWd = dY^T h: K runs over the tokens, every K block waits for its rows of the gathered dY
        dw_down = G.gemm(dybuf.local, h, a_mn=True, b_mn=True, k_ready=dy_ready, dependent=True, trigger=True)
        # (6) dWgu = [dg|du]^T X: K blocks wait for their rows of [dg|du]
        dw_gate_up = G.gemm(dgu, xbuf.local, a_mn=True, b_mn=True, k_ready=dgu_ready, dependent=True)
        return dx, dw_gate_up, dw_down


class _FusedTPFFNFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_gate_up, w_down, op: FusedTPFFN):
        ctx.op = op
        return op.forward(x, w_gate_up, w_down, save=True)

    @staticmethod
    def backward(ctx, dy):
        dx, dwgu, dwd = ctx.op.backward(dy)
        return dx, dwgu, dwd, None


def fused_tp_ffn(x, w_gate_up, w_down, op: FusedTPFFN):
    """Autograd entry point; ``op`` owns the symmetric workspaces."""
    return _FusedTPFFNFn.apply(x, w_gate_up, w_down, op)
