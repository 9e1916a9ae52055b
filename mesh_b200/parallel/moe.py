"""Expert-parallel routed MoE layer (softmax router, top-k, SwiGLU experts) on fused kernels.

Reference model: the GShard-style example ``examples/ep.py:15-70`` (router softmax -> top-k, slotting in token
order, capacity limit, batched expert SwiGLU, weighted combine) whose placement makes the compiler emit an
all-to-all (``examples/ep.py:74-85``).  Here the all-to-alls are fused into the dispatch and combine kernels
(peer stores / peer loads over the symmetric heap), the per-expert sizes never visit the host, and the expert
matmuls are descriptor-driven tcgen05 launches over compact per-expert row regions.

Forward:  router GEMM -> top-k -> count/slot -> plan -> dispatch(x) -> GLU GEMM -> down GEMM -> ready -> combine.
Backward: dispatch(w*dOut) + dots(<y, dOut>) -> dH GEMM (GLU backward epilogue) -> dW2 -> dX GEMM -> dW1 ->
          ready -> combine(dX) ; router gradient through softmax/top-k in PyTorch on the [tokens, experts] logits.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_uint32, c_void_p

import torch

from .. import _native
from ..ops import gemm as G
from ..ops.router import router_topk
from ..utils.status import status_block

MAX_RANKS = 8
DISPATCH_BLOCKS = 296


class _Plan(ctypes.Structure):
    _fields_ = [("counts", c_void_p), ("seq", c_uint32), ("rank", c_int), ("world", c_int), ("experts", c_int),
                ("cap_rows", c_int), ("d_model", c_int), ("d_ff", c_int), ("send_base", c_void_p), ("layout", c_void_p),
                ("tables", c_void_p * 6), ("n_tiles", c_void_p), ("max_tiles", c_int), ("status", c_void_p)]


class _Dispatch(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("tokens", c_int), ("k", c_int), ("d_model", c_int), ("idx", c_void_p), ("slot", c_void_p),
                ("send_base", c_void_p), ("scale", c_void_p), ("meta", c_void_p), ("local_experts", c_int),
                ("cap_rows", c_int), ("rank", c_int), ("world", c_int), ("recv", c_void_p * MAX_RANKS),
                ("arrived", c_void_p * MAX_RANKS), ("status", c_void_p)]


class _Combine(ctypes.Structure):
    _fields_ = [("tokens", c_int), ("k", c_int), ("d_model", c_int), ("local_experts", c_int), ("world", c_int),
                ("idx", c_void_p), ("meta", c_void_p), ("weight", c_void_p), ("src", c_void_p * MAX_RANKS),
                ("ready", c_void_p), ("ready_expect", c_uint32), ("out", c_void_p), ("dot_with", c_void_p),
                ("dots", c_void_p), ("status", c_void_p), ("cap_rows", c_int)]


def _s():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class EPMoE:
    """One MoE layer's expert-parallel machinery for a fixed (tokens per rank, d_model, d_ff, experts, k)."""

    def __init__(self, ctx, tokens: int, d_model: int, d_ff: int, experts: int, k: int, capacity_factor: float = 2.0):
        self.ctx = ctx
        self.rank, self.world = ctx.rank, ctx.world
        self.T, self.D, self.F, self.E, self.k = tokens, d_model, d_ff, experts, k
        assert experts % self.world == 0
        self.El = experts // self.world
        self.cap = int(-(-int(capacity_factor * tokens * k + 256 * self.El) // 256) * 256)
        heap, dev = ctx.heap, ctx.device
        self.dev = dev
        P = self.world
        # symmetric buffers: tokens in, expert outputs back (forward and backward each), counts, counters
        self.recv_x = heap.alloc((self.cap, d_model), torch.bfloat16)
        self.y = heap.alloc((self.cap, d_model), torch.bfloat16)
        self.recv_dy = heap.alloc((self.cap, d_model), torch.bfloat16)
        self.dx = heap.alloc((self.cap, d_model), torch.bfloat16)
        self.counts = heap.alloc((2 * P * experts * 2,), torch.int32)
        self.sig = heap.alloc_signals(8)           # 0: x arrived, 1: dy arrived, 2: y ready, 3: dx ready
        self.counts.local.zero_()
        torch.cuda.synchronize()
        ctx.rdv.barrier("moe-init")
        self.steps = 0
        mt = self.cap // 256 + self.El
        self.max_tiles = mt * max(-(-d_ff // 128), d_model // 256 + 1, -(-2 * d_ff // 256) * (d_model // 256)) + 64
        i32 = dict(dtype=torch.int32, device=dev)
        self.side = torch.cuda.Stream(dev)          # the router's backward runs beside the experts' (see backward)
        self.slot = torch.zeros(tokens * k, **i32)
        self.count_work = torch.zeros(int(_native.lib().mesh_moe_count_work_ints(c_int(tokens * k), c_int(experts))), **i32)
        self.meta = torch.zeros(tokens * k, **i32)
        self.send_base = torch.zeros(experts, **i32)
        self.layout = torch.zeros(3 * self.El + 2, **i32)
        self.tables = [torch.zeros((self.max_tiles, 8), **i32) for _ in range(6)]
        self.n_tiles = torch.zeros(6, **i32)
        self.h = torch.empty((self.cap, d_ff), dtype=torch.bfloat16, device=dev)
        self.gu = torch.empty((self.cap, 2 * d_ff), dtype=torch.bfloat16, device=dev)
        self.dgu = torch.empty((self.cap, 2 * d_ff), dtype=torch.bfloat16, device=dev)
        self.L = _native.lib()

    # ------------------------------------------------------------------ kernels
    def _grouped(self, table: int, A, B, D, *, M, N, K, a_mn=False, b_mn=False, epi=G.EPI_STORE, D2=None, aux=None,
                 b_up_rows=0, d_up_cols=0, a_ready=None, a_ready_value=0, b_rows=0, d_cols=0):
        g = _native.GemmArgs()
        g.A, g.B, g.D = A.data_ptr(), B.data_ptr(), D.data_ptr()
        g.M, g.N, g.K = M, N, K
        g.lda, g.ldb, g.ldd = A.stride(0), B.stride(0), D.stride(0)
        g.a_rows = A.shape[0]                     # stored rows (K-major: M bound; MN-major: K bound)
        g.b_rows = b_rows or B.shape[0]
        g.d_cols = d_cols or D.shape[1]
        g.d_rows = D.shape[0]
        g.a_mn, g.b_mn, g.epi, g.act = int(a_mn), int(b_mn), epi, 0
        g.b_up_rows, g.d_up_cols = b_up_rows, d_up_cols
        if D2 is not None:
            g.D2, g.ldd2, g.d2_cols = D2.data_ptr(), D2.stride(0), D2.shape[1]
        if aux is not None:
            g.aux, g.ld_aux = aux.data_ptr(), aux.stride(0)
        if a_ready is not None:
            g.a_ready, g.a_ready_value, g.a_ready_rows = a_ready, a_ready_value, 1 << 30
        g.status = status_block(self.dev).data_ptr()
        g.world = 1
        g.tiles, g.n_tiles_dev, g.max_tiles = self.tables[table].data_ptr(), self.n_tiles[table:].data_ptr(), self.max_tiles
        g.pair, g.tile_n = 1, 256
        G._launch(g)

    def _dispatch(self, x, scale, recv, sig_index):
        d = _Dispatch()
        d.x, d.tokens, d.k, d.d_model = x.data_ptr(), self.T, self.k, self.D
        d.idx, d.slot, d.send_base = self.idx.data_ptr(), self.slot.data_ptr(), self.send_base.data_ptr()
        d.scale = 0 if scale is None else scale.data_ptr()
        d.meta = self.meta.data_ptr()
        d.local_experts, d.cap_rows, d.rank, d.world = self.El, self.cap, self.rank, self.world
        for r in range(self.world):
            d.recv[r] = recv.ptr(r)
            d.arrived[r] = self.sig.ptr(r) + 4 * sig_index
        d.status = status_block(self.dev).data_ptr()
        _native.check(self.L.mesh_moe_dispatch(ctypes.byref(d), _s()), "mesh_moe_dispatch")
        _native.count_launch()

    def _signal(self, sig_index):
        arr = (c_void_p * MAX_RANKS)(*[c_void_p(self.sig.ptr(r) + 4 * sig_index) if r < self.world else c_void_p(0) for r in range(MAX_RANKS)])
        _native.check(self.L.mesh_moe_signal(c_int(self.world), arr, _s()), "mesh_moe_signal")
        _native.count_launch()

    def _combine(self, src, sig_index, weight, out, dot_with=None, dots=None):
        c = _Combine()
        c.tokens, c.k, c.d_model, c.local_experts, c.world = self.T, self.k, self.D, self.El, self.world
        c.idx, c.meta = self.idx.data_ptr(), self.meta.data_ptr()
        c.weight = 0 if weight is None else weight.data_ptr()
        for r in range(self.world):
            c.src[r] = src.ptr(r)
        c.ready, c.ready_expect = self.sig.ptr() + 4 * sig_index, self.world * self.steps
        c.out = 0 if out is None else out.data_ptr()
        c.dot_with = 0 if dot_with is None else dot_with.data_ptr()
        c.dots = 0 if dots is None else dots.data_ptr()
        c.status = status_block(self.dev).data_ptr()
        c.cap_rows = self.cap
        _native.check(self.L.mesh_moe_combine(ctypes.byref(c), _s()), "mesh_moe_combine")
        _native.count_launch()

    # ------------------------------------------------------------------ phase timeline (benchmarks)
    timeline: list | None = None      # set to [] to record a CUDA event after every phase of forward / backward

    def _mark(self, name: str) -> None:
        if _native.nvtx.enabled:                  # an NVTX marker at the end of every phase
            torch.cuda.nvtx.mark("moe: " + name)
        if self.timeline is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.timeline.append((name, e))

    @staticmethod
    def phases(timeline: list) -> list:
        """``[(phase, microseconds)]`` from a recorded timeline (after a synchronize): the time between consecutive
        marks, i.e. the kernels of that phase as the stream ran them."""
        return [(b[0], a[1].elapsed_time(b[1]) * 1e3) for a, b in zip(timeline, timeline[1:])]

    # ------------------------------------------------------------------ forward / backward
    def forward(self, x, w_router, w1, w2, bias=None):
        """x [T, D] bf16; w_router [E, D]; w1 [El*2F, D] (per expert: gate rows then up rows); w2 [El*D, F]."""
        T, D, F, k = self.T, self.D, self.F, self.k
        self.steps += 1
        self._mark("start")
        logits = G.gemm(x, w_router)                                            # [T, E]
        weights, idx = router_topk(logits, k, bias, renorm=True)
        self._mark("router")
        self.idx = idx.reshape(-1).contiguous()
        arr = (c_void_p * MAX_RANKS)(*[c_void_p(self.counts.ptr(r)) if r < self.world else c_void_p(0) for r in range(MAX_RANKS)])
        _native.check(self.L.mesh_moe_count(c_void_p(self.idx.data_ptr()), c_int(T * k), c_void_p(self.slot.data_ptr()),
                                            c_int(self.E), c_int(self.rank), c_int(self.world), arr, c_uint32(self.steps),
                                            c_void_p(self.count_work.data_ptr()), _s()),
                      "mesh_moe_count")
        p = _Plan()
        p.counts, p.seq, p.rank, p.world, p.experts = self.counts.ptr(), self.steps, self.rank, self.world, self.E
        p.cap_rows, p.d_model, p.d_ff = self.cap, D, F
        p.send_base, p.layout = self.send_base.data_ptr(), self.layout.data_ptr()
        for i in range(6):
            p.tables[i] = self.tables[i].data_ptr()
        p.n_tiles, p.max_tiles, p.status = self.n_tiles.data_ptr(), self.max_tiles, status_block(self.dev).data_ptr()
        _native.check(self.L.mesh_moe_plan(ctypes.byref(p), _s()), "mesh_moe_plan")
        _native.check(self.L.mesh_moe_zero_pad(c_void_p(self.recv_x.ptr()), c_void_p(self.layout.data_ptr()), c_int(self.El),
                                               c_int(D), _s()), "mesh_moe_zero_pad")
        _native.count_launch(3)
        self._mark("count+plan+pad")
        self._dispatch(x, None, self.recv_x, 0)
        self._mark("dispatch")
        expect = self.world * DISPATCH_BLOCKS * self.steps
        rx = self.recv_x.local
        self._grouped(0, rx, w1, self.h, M=self.cap, N=F, K=D, epi=G.EPI_GLU_FWD, D2=self.gu, b_up_rows=F, d_up_cols=F,
                      a_ready=self.sig.ptr() + 0, a_ready_value=expect)
        self._mark("experts glu")
        self._grouped(1, self.h, w2, self.y.local, M=self.cap, N=D, K=F)
        self._mark("experts down")
        self._signal(2)
        out = torch.empty((T, D), dtype=torch.bfloat16, device=self.dev)
        self._combine(self.y, 2, weights.reshape(-1), out)
        self._mark("combine")
        self._saved = (x, w_router, w1, w2, logits, weights, bias)
        return out

    def backward(self, dout):
        x, w_router, w1, w2, logits, weights, bias = self._saved
        T, D, F, k = self.T, self.D, self.F, self.k
        dout = dout.contiguous()
        # Gradients of the routing weights, <expert output row, dOut[t]> (reads the forward's y on the peers), and
        # the router's own backward need nothing of the expert backward: they run on a second stream beside it (the
        # pull of y is inbound NVLink traffic while the dispatch of dOut is outbound) and join at the end.
        import os
        overlap = os.environ.get("MESH_MOE_OVERLAP", "1") != "0" and self.timeline is None
        main = torch.cuda.current_stream(self.dev)
        side = self.side if overlap else main
        dots = torch.empty((T, k), dtype=torch.float32, device=self.dev)
        self._mark("bwd start")

        def router_backward():
            self._combine(self.y, 2, None, None, dot_with=dout, dots=dots.view(-1))
            self._mark("bwd weight dots")
            # router: weights = renormalised top-k of softmax(logits + bias)
            lg = logits.float().detach().requires_grad_(True)
            p = torch.softmax(lg + (bias.float() if bias is not None else 0.0), dim=-1)
            sel = torch.gather(p, 1, self.idx.view(T, k).long())
            wn = sel / sel.sum(-1, keepdim=True)
            kept = (self.meta.view(T, k) >= 0).float()
            (wn * dots * kept).sum().backward()
            dlogits = lg.grad.to(torch.bfloat16)
            dxr = G.gemm(dlogits, w_router, b_mn=True)
            dwr = G.gemm(dlogits, x, a_mn=True, b_mn=True) if (dlogits.shape[1] % 64 == 0 and x.shape[1] % 64 == 0) else \
                (dlogits.float().T @ x.float()).to(torch.bfloat16)
            self._mark("bwd router")
            return dxr, dwr

        if overlap:
            side.wait_stream(main)
            with torch.cuda.stream(side):
                dx_router, dw_router = router_backward()
        else:
            dx_router, dw_router = router_backward()
        _native.check(self.L.mesh_moe_zero_pad(c_void_p(self.recv_dy.ptr()), c_void_p(self.layout.data_ptr()), c_int(self.El),
                                               c_int(D), _s()), "mesh_moe_zero_pad")
        self._dispatch(dout, weights.reshape(-1).contiguous(), self.recv_dy, 1)
        self._mark("bwd dispatch")
        expect = self.world * DISPATCH_BLOCKS * self.steps
        rdy, rx = self.recv_dy.local, self.recv_x.local
        self._grouped(2, rdy, w2, self.dgu, M=self.cap, N=F, K=D, b_mn=True, epi=G.EPI_GLU_BWD, aux=self.gu, d_up_cols=F,
                      a_ready=self.sig.ptr() + 4, a_ready_value=expect, d_cols=2 * F)
        self._mark("bwd dH glu")
        dw2 = torch.zeros_like(w2)
        self._grouped(4, rdy, self.h, dw2, M=D, N=F, K=self.cap, a_mn=True, b_mn=True)
        self._mark("bwd dW2")
        self._grouped(3, self.dgu, w1, self.dx.local, M=self.cap, N=D, K=2 * F, b_mn=True)
        self._mark("bwd dX")
        dw1 = torch.zeros_like(w1)
        self._grouped(5, self.dgu, rx, dw1, M=2 * F, N=D, K=self.cap, a_mn=True, b_mn=True)
        self._mark("bwd dW1")
        self._signal(3)
        dx = torch.empty((T, D), dtype=torch.bfloat16, device=self.dev)
        self._combine(self.dx, 3, None, dx)
        self._mark("bwd combine")
        if overlap:
            main.wait_stream(side)
            for t in (dx_router, dw_router, dots):
                t.record_stream(main)
        dx = dx + dx_router
        return dx, dw_router, dw1, dw2


def moe_reference(x, w_router, w1_all, w2_all, k, bias=None):
    """Dense fp32 statement of the same layer with every expert's weights (no capacity limit): the oracle.
    ``w1_all [E, 2F, D]``, ``w2_all [E, D, F]``."""
    xf = x.float()
    logits = (xf @ w_router.float().T).to(torch.bfloat16).float()
    p = torch.softmax(logits + (bias.float() if bias is not None else 0.0), -1)
    w, idx = torch.topk(p, k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    F = w1_all.shape[1] // 2
    out = torch.zeros_like(xf)
    for e in range(w1_all.shape[0]):
        tok, j = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = xf[tok]
        h = torch.nn.functional.silu(xe @ w1_all[e, :F].float().T) * (xe @ w1_all[e, F:].float().T)
        out.index_add_(0, tok, (h @ w2_all[e].float().T) * w[tok, j][:, None])
    return out
