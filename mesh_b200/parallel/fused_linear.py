"""Column- and row-parallel linear layers over sequence-sharded activations, each direction one fused kernel.

The tensor-parallel attention projections have the same structure as the FFN halves (the reference's ``megatron()``
placement cuts ``wq, wk, wv`` by rows and ``wo`` by columns, examples/parallel.py:77-89, and its compiler puts an
all-gather before the first and a reduce after the second, compiler/mesh_compiler/placement.py:250-340, :812-834):

* :class:`FusedColumnLinear` - ``y = all_gather(x) W^T``: the kernel pushes this rank's token rows to every peer's
  gathered buffer while its tensor-core tiles start on the rows that have arrived.  Backward: ``dx`` is a GEMM whose
  epilogue scatters tiles to the owners of the token rows, which sum them (reduce-scatter); ``dW = dy^T X`` reuses
  the gathered ``X``.
* :class:`FusedRowLinear` - ``y = reduce_scatter(h W^T)``: GEMM with the scattering epilogue.  Backward: all-gather of
  ``dy`` fused into the ``dh = dY W`` GEMM; ``dW = dY^T h`` reuses the gathered ``dY``.

The landing zones are the double-buffered ones of ``tp_ffn.py`` (monotonic counters, no barriers between steps).
"""
from __future__ import annotations

import torch

from .. import _native
from ..ops import gemm as G
from ..utils.status import status_block
from .tp_ffn import BM, _Gathered, _Scattered, shared_zone


class _FusedBase:
    def __init__(self, heap, tokens: int, d_in: int, d_out: int):
        self.heap, self.rank, self.world = heap, heap.rank, heap.world
        P = self.world
        if tokens % (P * BM):
            raise ValueError(f"tokens ({tokens}) must be a multiple of world*128")
        if d_in % 64 or d_out % 64:
            raise ValueError("feature sizes must be multiples of 64")
        self.M, self.rows = tokens, tokens // P

    def _args(self, dev) -> _native.GemmArgs:
        g = _native.GemmArgs()
        g.status = status_block(dev).data_ptr()
        g.rank, g.world = self.rank, self.world
        return g

    def _gather_args(self, g, zone: _Gathered, src: torch.Tensor, width: int):
        buf, flags, expect = zone.next()
        g.A, g.lda, g.a_rows = buf.ptr(), width, self.M
        g.a_ready, g.a_ready_value, g.a_ready_rows = flags.ptr(), expect, BM
        g.m_rotate = self.rank * (self.rows // BM)
        g.ag_src, g.ag_rows_per_rank, g.ag_ld = src.data_ptr(), self.rows, width
        g.ag_split = zone.split
        for r in range(self.world):
            g.ag_dst[r] = buf.ptr(r)
            g.ag_flags[r] = flags.ptr(r)
        return buf

    def _scatter_args(self, g, zone: _Scattered, out: torch.Tensor):
        buf, count, expect = zone.next()
        g.epi = G.EPI_SCATTER
        g.tile_n = zone.tile_n
        for r in range(self.world):
            g.rs_recv[r] = buf.ptr(r)
            g.rs_count[r] = count.ptr(r)
        g.rs_expect, g.rs_out, g.rs_rows_per_rank = expect, (0 if out is None else out.data_ptr()), self.rows
        g.m_rotate = ((self.rank + 1) % self.world) * (self.rows // BM)
        return zone


class FusedColumnLinear(_FusedBase):
    """``w``: this rank's ``[N_local, D]`` rows of the weight."""

    def __init__(self, heap, tokens: int, d_in: int, n_local: int, in_flight: int = 1):
        super().__init__(heap, tokens, d_in, n_local)
        self.D, self.N = d_in, n_local
        self.x_full = _Gathered(heap, tokens, d_in, copies=in_flight + 1)   # X is read again by the backward pass
        self.dx_recv = shared_zone(heap, _Scattered, self.world, self.rows, d_in)

    def forward(self, x: torch.Tensor, w: torch.Tensor):
        dev = x.device
        y = torch.empty((self.M, self.N), dtype=torch.bfloat16, device=dev)
        g = self._args(dev)
        xbuf = self._gather_args(g, self.x_full, x, self.D)
        g.B, g.ldb, g.b_rows = w.data_ptr(), w.stride(0), self.N
        g.M, g.N, g.K = self.M, self.N, self.D
        g.epi = G.EPI_STORE
        g.D, g.ldd, g.d_cols = y.data_ptr(), self.N, self.N
        G._launch(g)
        return y, xbuf

    def backward(self, dy: torch.Tensor, w: torch.Tensor, xbuf):
        dev = dy.device
        dy = dy.contiguous()
        dx = torch.empty((self.rows, self.D), dtype=torch.bfloat16, device=dev)
        g = self._args(dev)
        g.A, g.lda, g.a_rows = dy.data_ptr(), self.N, self.M
        g.B, g.ldb, g.b_mn = w.data_ptr(), w.stride(0), 1            # dx = dy W: W [N, D] read as [K = N rows, D cols]
        g.M, g.N, g.K = self.M, self.D, self.N
        self._scatter_args(g, self.dx_recv, dx)
        G._launch(g)
        dw = G.gemm(dy, xbuf.local, a_mn=True, b_mn=True)            # [N, D] = dy^T X
        return dx, dw


class FusedRowLinear(_FusedBase):
    """``w``: this rank's ``[D, K_local]`` columns of the weight."""

    def __init__(self, heap, tokens: int, k_local: int, d_out: int):
        super().__init__(heap, tokens, k_local, d_out)
        self.K, self.D = k_local, d_out
        self.y_recv = shared_zone(heap, _Scattered, self.world, self.rows, d_out)
        self.dy_full = shared_zone(heap, _Gathered, tokens, d_out)

    def forward(self, h: torch.Tensor, w: torch.Tensor):
        dev = h.device
        y = torch.empty((self.rows, self.D), dtype=torch.bfloat16, device=dev)
        g = self._args(dev)
        g.A, g.lda, g.a_rows = h.data_ptr(), h.stride(0), self.M
        g.B, g.ldb, g.b_rows = w.data_ptr(), w.stride(0), self.D
        g.M, g.N, g.K = self.M, self.D, self.K
        self._scatter_args(g, self.y_recv, y)
        G._launch(g)
        return y

    def backward(self, dy: torch.Tensor, h: torch.Tensor, w: torch.Tensor):
        dev = dy.device
        dy = dy.contiguous()
        dh = torch.empty((self.M, self.K), dtype=torch.bfloat16, device=dev)
        g = self._args(dev)
        dybuf = self._gather_args(g, self.dy_full, dy, self.D)
        g.B, g.ldb, g.b_mn = w.data_ptr(), w.stride(0), 1            # dh = dY W: W [D, K] read as [K = D rows, K cols]
        g.M, g.N, g.K = self.M, self.K, self.D
        g.epi = G.EPI_STORE
        g.D, g.ldd, g.d_cols = dh.data_ptr(), self.K, self.K
        G._launch(g)
        dw = G.gemm(dybuf.local, h, a_mn=True, b_mn=True)            # [D, K] = dY^T h
        return dh, dw


class _ColumnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, op: FusedColumnLinear):
        y, xbuf = op.forward(x.contiguous(), w)
        ctx.op, ctx.xbuf = op, xbuf
        ctx.save_for_backward(w)
        return y

    @staticmethod
    def backward(ctx, dy):
        (w,) = ctx.saved_tensors
        dx, dw = ctx.op.backward(dy, w, ctx.xbuf)
        return dx, dw, None


class _RowFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, op: FusedRowLinear):
        h = h.contiguous()
        ctx.op = op
        ctx.save_for_backward(h, w)
        return op.forward(h, w)

    @staticmethod
    def backward(ctx, dy):
        h, w = ctx.saved_tensors
        dh, dw = ctx.op.backward(dy, h, w)
        return dh, dw, None


def column_linear(x, w, op: FusedColumnLinear):
    """``x``: this rank's ``[tokens/world, D]`` rows -> ``[tokens, N_local]`` for all tokens."""
    return _ColumnFn.apply(x, w, op)


def row_linear(h, w, op: FusedRowLinear):
    """``h [tokens, K_local]`` -> this rank's ``[tokens/world, D]`` rows of the summed product."""
    return _RowFn.apply(h, w, op)


class FusedRowLinearAllReduce(_FusedBase):
    """``y = all_reduce(h W^T)`` for layers whose activations are not cut over the tokens (plain Megatron tensor
    parallelism, the row-parallel half: examples/parallel.py:84-89 of the reference, whose compiler emits a reduce
    there, compiler/mesh_compiler/placement.py:812-834).

    ONE kernel: the GEMM's epilogue scatters the partial tiles to the owners of their token rows; as soon as an owner
    has summed a tile of its rows it stores the sum into every rank's full output (peer stores) and raises that rank's
    counter; the kernel ends on every rank when all other ranks' tiles have arrived.  The partial products never make
    a round trip through HBM before they cross NVLink, and the gathering half starts while later tiles are still being
    multiplied.  ``MESH_FUSED_AR=0`` runs the older composition (the same scattering GEMM, then the communicator's
    all-gather kernel).  Backward: ``dy`` is whole on every rank, so ``dh = dy W`` and ``dW = dy^T h`` are local."""

    def __init__(self, heap, comm, tokens: int, k_local: int, d_out: int):
        import os
        super().__init__(heap, tokens, k_local, d_out)
        self.row = FusedRowLinear(heap, tokens, k_local, d_out)
        self.comm, self.D, self.K = comm, d_out, k_local
        self.one_kernel = os.environ.get("MESH_FUSED_AR", "1") != "0"
        if self.one_kernel:
            # full outputs [tokens, D], two of them used in turn (a rank can be one use ahead of a peer), and one
            # arrival counter each; counters only grow
            self.full = [heap.alloc((tokens, d_out), torch.bfloat16) for _ in range(2)]
            self.flag = [heap.alloc_signals(1) for _ in range(2)]
            self.uses = [0, 0]
            self.turn = 0

    def forward(self, h: torch.Tensor, w: torch.Tensor, copy: bool = True) -> torch.Tensor:
        """``copy=False`` returns the landing buffer itself, which is overwritten two calls later."""
        if not self.one_kernel:
            mine = self.row.forward(h, w)                                 # [tokens / world, D]: summed over the ranks
            full = torch.empty((self.M, self.D), dtype=mine.dtype, device=mine.device)
            self.comm.all_gather(full, mine)
            return full
        dev = h.device
        par = self.turn & 1
        self.turn += 1
        self.uses[par] += 1
        g = self._args(dev)
        g.A, g.lda, g.a_rows = h.data_ptr(), h.stride(0), self.M
        g.B, g.ldb, g.b_rows = w.data_ptr(), w.stride(0), self.D
        g.M, g.N, g.K = self.M, self.D, self.K
        zone = self._scatter_args(g, self.row.y_recv, None)
        n_tiles = (self.D + zone.tile_n - 1) // zone.tile_n
        for r in range(self.world):
            g.ar_out[r] = self.full[par].ptr(r)
            g.ar_flag[r] = self.flag[par].ptr(r)
        g.ar_expect = ((self.world - 1) * (self.rows // BM) * n_tiles * self.uses[par]) & 0xFFFFFFFF
        G._launch(g)
        out = self.full[par].local.view(self.M, self.D)
        return out.clone() if copy else out

    def backward(self, dy: torch.Tensor, h: torch.Tensor, w: torch.Tensor):
        dy = dy.contiguous()
        dh = G.gemm(dy, w, b_mn=True)                                     # [tokens, K_local] = dy W, W [D, K] read as [K = D, N = K_local]
        dw = G.gemm(dy, h, a_mn=True, b_mn=True)                          # [D, K_local] = dy^T h
        return dh, dw


class _RowARFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, op: FusedRowLinearAllReduce):
        h = h.contiguous()
        ctx.op = op
        ctx.save_for_backward(h, w)
        return op.forward(h, w)

    @staticmethod
    def backward(ctx, dy):
        h, w = ctx.saved_tensors
        dh, dw = ctx.op.backward(dy, h, w)
        return dh, dw, None


def row_linear_all_reduce(h, w, op: FusedRowLinearAllReduce):
    """``h [tokens, K_local]`` -> ``[tokens, D]``, the product summed over the ranks, whole on every rank."""
    return _RowARFn.apply(h, w, op)
