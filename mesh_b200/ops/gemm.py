"""bf16 GEMMs on the 5th-generation tensor cores (tcgen05 + TMEM, TMA-fed) and their fused forms.

All matrices are row-major ``torch.bfloat16`` CUDA tensors.  ``gemm(a, b)`` computes
``a @ b.T`` like ``torch.nn.functional.linear``; the ``*_mn`` flags say that an operand is stored
transposed (``[K, rows]``), which lets dgrad and wgrad reuse the same kernel with no transposed
copies.  The GLU helpers fuse the SwiGLU / GeGLU pointwise math into the GEMM epilogues.

Reference semantics: contraction ``compiler/mesh_compiler/operations.py:1191-1272``; SwiGLU FFN of
``examples/parallel.py:44-51``; GeGLU-tanh of ``examples/engines.py:44``.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from ..utils.status import status_block

EPI_STORE, EPI_GLU_FWD, EPI_GLU_BWD, EPI_SCATTER = 0, 1, 2, 3
ACT = {"silu": 0, "swiglu": 0, "gelu_tanh": 1, "geglu": 1}


def _check2d(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name}: expected a 2-D row-major bf16 CUDA tensor, got {t.dtype} {tuple(t.shape)} {t.stride()}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_trace: list | None = None


class trace:
    """``with trace() as t:`` records a CUDA-event pair around every GEMM launch of the block;
    ``t.report()`` gives ``[(label, microseconds)]`` (after a synchronize).  For per-kernel breakdowns: meaningful only
    with launches that do not overlap (``MESH_GEMM_CHAIN=0``)."""

    def __enter__(self):
        global _trace
        self.items = []
        _trace = self.items
        return self

    def __exit__(self, *exc):
        global _trace
        _trace = None

    def report(self):
        torch.cuda.synchronize()
        return [(label, e0.elapsed_time(e1) * 1e3) for label, e0, e1 in self.items]


def _label(a: _native.GemmArgs) -> str:
    epi = {EPI_STORE: "store", EPI_GLU_FWD: "glu_fwd", EPI_GLU_BWD: "glu_bwd", EPI_SCATTER: "reduce_scatter"}[a.epi]
    pre = "all_gather+" if a.ag_src else ""
    return f"{pre}gemm[{a.M}x{a.N}x{a.K}{' A^T' if a.a_mn else ''}{' B^T' if a.b_mn else ''}]->{epi}"


def _launch(args: _native.GemmArgs) -> None:
    if _trace is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    if _native.nvtx.enabled:
        with _native.nvtx(_label(args)):
            rc = _native.lib().mesh_gemm_bf16(ctypes.byref(args), ctypes.c_void_p(_stream()))
    else:
        rc = _native.lib().mesh_gemm_bf16(ctypes.byref(args), ctypes.c_void_p(_stream()))
    _native.check(rc, "mesh_gemm_bf16")
    _native.count_launch()
    if _trace is not None:
        e1.record()
        _trace.append((_label(args), e0, e1))


def _base_args(a: torch.Tensor, b: torch.Tensor, a_mn: bool, b_mn: bool) -> tuple[_native.GemmArgs, int, int, int]:
    _check2d(a, "a")
    _check2d(b, "b")
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"contraction sizes differ: {K} vs {Kb}")
    g = _native.GemmArgs()
    g.A, g.B = a.data_ptr(), b.data_ptr()
    g.M, g.N, g.K = M, N, K
    g.lda, g.ldb = a.stride(0), b.stride(0)
    g.a_mn, g.b_mn = int(a_mn), int(b_mn)
    g.a_rows = 0 if a_mn else a.shape[0]
    g.b_rows = 0 if b_mn else b.shape[0]
    g.status = status_block(a.device).data_ptr()
    g.world = 1
    return g, M, N, K


PDL_DEPENDENT, PDL_TRIGGER = 1, 2
BM = 128
EPI_WARPS = 4


class Done:
    """Completion counters of a chain of launches: one per 128 rows of a matrix that one kernel writes and the next
    launches of the stream read while the writer's last tiles are still running (see ``Params`` in
    csrc/gemm/gemm_sm100.cuh).  Counters only grow; every use of the chain expects ``tiles x 4`` more arrivals."""

    _cache: dict = {}

    def __init__(self, device, row_blocks: int):
        self.flags = torch.zeros(row_blocks, dtype=torch.int32, device=device)
        self.total = 0

    @classmethod
    def get(cls, device, row_blocks: int, tag: str) -> "Done":
        key = (torch.device(device).index, row_blocks, tag)
        if key not in cls._cache:
            cls._cache[key] = cls(device, row_blocks)
        return cls._cache[key]

    def produce(self, n_tiles: int) -> int:
        """The writer's launch: returns the counter value that means "this launch has written the row block"."""
        self.total = (self.total + n_tiles * EPI_WARPS) & 0x7FFFFFFF
        return self.total

    def ptr(self) -> int:
        return self.flags.data_ptr()


def chain(g: _native.GemmArgs, *, d_done: Done | None = None, a_ready=None, k_ready=None, dependent: bool = False,
          trigger: bool = False) -> None:
    """Dataflow attributes of one launch.  ``a_ready`` / ``k_ready``: ``(pointer, value, rows)``."""
    if d_done is not None:
        g.d_done = d_done.ptr()
    if a_ready is not None:
        g.a_ready, g.a_ready_value, g.a_ready_rows = a_ready
    if k_ready is not None:
        g.k_ready, g.k_ready_value, g.k_ready_rows = k_ready
    g.pdl = (PDL_DEPENDENT if dependent else 0) | (PDL_TRIGGER if trigger else 0)


def chaining() -> bool:
    """Consecutive GEMMs of a layer overlap (dependent launches + row-block counters) unless ``MESH_GEMM_CHAIN=0``."""
    import os
    return os.environ.get("MESH_GEMM_CHAIN", "1") != "0"


def tile_n_for(M: int, N: int) -> int:
    return _native.lib().mesh_gemm_choose_tile_n(M, N, 0)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, num_ctas: int = 0, tile_n: int = 0, pair: int = 0, **flow) -> torch.Tensor:
    """``out[M,N] = A[M,K] @ B[N,K]^T`` with fp32 accumulation.

    ``a_mn``: ``a`` is stored ``[K, M]``;  ``b_mn``: ``b`` is stored ``[K, N]``.  ``flow``: see :func:`chain`.
    """
    g, M, N, K = _base_args(a, b, a_mn, b_mn)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    _check2d(out, "out")
    g.D, g.ldd, g.d_cols = out.data_ptr(), out.stride(0), out.shape[1]
    g.epi = EPI_STORE
    g.num_ctas, g.tile_n, g.pair = num_ctas, tile_n, pair
    if flow:
        chain(g, **flow)
    _launch(g)
    return out


def gemm_q(a: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, *, out: torch.Tensor | None = None,
           num_ctas: int = 0, tile_n: int = 0, pair: int = 0) -> torch.Tensor:
    """``out[M, N] = a[M, K] @ W[N, K]^T`` with ``W`` group-quantised: ``codes`` uint8 ``[N, K/2]`` (4-bit,
    :func:`mesh_b200.ops.decode.quantize_w4`) or ``[N, K]`` (8-bit, ``quantize_w8``) and ``scales`` fp16 ``[N, K/64]``.

    The codes are dequantised in registers by four extra warps of the GEMM kernel and written straight into the
    tensor cores' shared-memory stages: the bf16 matrix never exists in global memory (K13 of the reference's operation
    table; its coded weights are decoded the same way, compiler/mesh_compiler/operations.py:6996-7040)."""
    _check2d(a, "a")
    if codes.dtype != torch.uint8 or scales.dtype != torch.float16 or not codes.is_contiguous() or not scales.is_contiguous():
        raise ValueError("gemm_q: codes must be contiguous uint8 and scales contiguous fp16")
    M, K = a.shape
    N = codes.shape[0]
    bits = 8 if codes.shape[1] == K else 4
    if bits == 4 and codes.shape[1] * 2 != K:
        raise ValueError(f"gemm_q: codes of width {codes.shape[1]} do not fit K = {K} in 4 or 8 bits")
    if K % 64 or tuple(scales.shape) != (N, K // 64):
        raise ValueError("gemm_q: K must be a multiple of 64 with one scale per 64 inputs")
    g = _native.GemmArgs()
    g.A, g.B, g.b_scales, g.b_bits = a.data_ptr(), codes.data_ptr(), scales.data_ptr(), bits
    g.M, g.N, g.K = M, N, K
    g.lda, g.ldb = a.stride(0), K
    g.a_rows, g.b_rows = M, N
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    _check2d(out, "out")
    g.D, g.ldd, g.d_cols = out.data_ptr(), out.stride(0), out.shape[1]
    g.epi = EPI_STORE
    g.status = status_block(a.device).data_ptr()
    g.world = 1
    g.num_ctas, g.tile_n, g.pair = num_ctas, tile_n, pair
    _launch(g)
    return out


def glu_fwd(x: torch.Tensor, w_gate_up: torch.Tensor, *, act: str = "silu", save_gu: bool = True,
            out: torch.Tensor | None = None, gu: torch.Tensor | None = None, **flow):
    """``act(x @ Wg^T) * (x @ Wu^T)`` where ``w_gate_up = [Wg; Wu]`` is ``[2F, K]``.

    Returns ``(h[M,F], gu[M,2F] or None)``; ``gu = [g | u]`` is what the backward pass needs.
    """
    _check2d(x, "x")
    _check2d(w_gate_up, "w_gate_up")
    F2, K = w_gate_up.shape
    F = F2 // 2
    M = x.shape[0]
    g = _native.GemmArgs()
    g.A, g.B = x.data_ptr(), w_gate_up.data_ptr()
    g.M, g.N, g.K = M, F, K
    g.lda, g.ldb = x.stride(0), w_gate_up.stride(0)
    g.a_rows, g.b_rows = M, F2
    g.b_up_rows = F
    g.epi, g.act = EPI_GLU_FWD, ACT[act]
    if out is None:
        out = torch.empty((M, F), dtype=torch.bfloat16, device=x.device)
    g.D, g.ldd, g.d_cols = out.data_ptr(), out.stride(0), F
    if save_gu:
        if gu is None:
            gu = torch.empty((M, F2), dtype=torch.bfloat16, device=x.device)
        g.D2, g.ldd2, g.d2_cols, g.d_up_cols = gu.data_ptr(), gu.stride(0), F2, F
    else:
        gu = None
    g.status = status_block(x.device).data_ptr()
    g.world = 1
    if flow:
        chain(g, **flow)
    _launch(g)
    return out, gu


def glu_bwd(dy: torch.Tensor, w_down: torch.Tensor, gu: torch.Tensor, *, act: str = "silu",
            out: torch.Tensor | None = None, tile_n: int = 0, **flow) -> torch.Tensor:
    """Backward of the GLU through the down projection in one kernel.

    ``dH = dy @ w_down`` (``w_down`` is ``[D, F]``, used MN-major) and the epilogue turns it into
    ``[dg | du]`` (``[M, 2F]``) using the saved ``gu = [g | u]``.
    """
    _check2d(dy, "dy")
    _check2d(w_down, "w_down")
    _check2d(gu, "gu")
    M, D = dy.shape
    D2, F = w_down.shape
    if D2 != D or gu.shape != (M, 2 * F):
        raise ValueError("glu_bwd: shape mismatch")
    g = _native.GemmArgs()
    g.A, g.B = dy.data_ptr(), w_down.data_ptr()
    g.M, g.N, g.K = M, F, D
    g.lda, g.ldb = dy.stride(0), w_down.stride(0)
    g.a_rows = M
    g.b_mn = 1
    g.epi, g.act = EPI_GLU_BWD, ACT[act]
    g.aux, g.ld_aux = gu.data_ptr(), gu.stride(0)
    g.d_up_cols = F
    if out is None:
        out = torch.empty((M, 2 * F), dtype=torch.bfloat16, device=dy.device)
    g.D, g.ldd, g.d_cols = out.data_ptr(), out.stride(0), 2 * F
    g.status = status_block(dy.device).data_ptr()
    g.world = 1
    g.tile_n = tile_n
    if flow:
        chain(g, **flow)
    _launch(g)
    return out


class _Linear(torch.autograd.Function):
    """``y = x @ w^T`` with dgrad/wgrad on the same tcgen05 kernel (no transposes materialised)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w)
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(x.shape)          # [M,N] x [N,K] stored [K=N, cols=K]
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True)               # dy^T x : [N, K]
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _Linear.apply(x, w)


class _GluFFN(torch.autograd.Function):
    """Whole gated FFN ``(act(x Wg^T) * (x Wu^T)) Wd^T`` in 2 forward and 4 backward kernels."""

    @staticmethod
    def forward(ctx, x, w_gate_up, w_down, act):
        x2 = x.reshape(-1, x.shape[-1])
        M, F = x2.shape[0], w_gate_up.shape[0] // 2
        if chaining():
            # the down projection starts during the last wave of the gate/up GEMM and reads h row block by row block
            done = Done.get(x2.device, (M + BM - 1) // BM, "glu.h")
            h, gu = glu_fwd(x2, w_gate_up, act=act, save_gu=True, d_done=done, trigger=True)
            y = gemm(h, w_down, a_ready=(done.ptr(), done.produce((F + 127) // 128), BM), dependent=True)
        else:
            h, gu = glu_fwd(x2, w_gate_up, act=act, save_gu=True)
            y = gemm(h, w_down)
        ctx.save_for_backward(x2, w_gate_up, w_down, h, gu)
        ctx.act = act
        ctx.xshape = x.shape
        return y.reshape(*x.shape[:-1], w_down.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w_gate_up, w_down, h, gu = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        if chaining():
            M, F = dy2.shape[0], w_down.shape[1]
            done = Done.get(dy2.device, (M + BM - 1) // BM, "glu.dgu")
            bn = tile_n_for(M, F)
            dgu = glu_bwd(dy2, w_down, gu, act=ctx.act, tile_n=bn, d_done=done, trigger=True)       # [M, 2F]
            ready = (done.ptr(), done.produce((F + bn - 1) // bn), BM)
            dx = gemm(dgu, w_gate_up, b_mn=True, a_ready=ready, dependent=True, trigger=True).reshape(ctx.xshape)
            dw_down = gemm(dy2, h, a_mn=True, b_mn=True, dependent=True, trigger=True)          # reads nothing of the chain
            dw_gate_up = gemm(dgu, x2, a_mn=True, b_mn=True, k_ready=ready, dependent=True)      # [2F, D]
            return dx, dw_gate_up, dw_down, None
        dgu = glu_bwd(dy2, w_down, gu, act=ctx.act)                 # [M, 2F]
        dw_down = gemm(dy2, h, a_mn=True, b_mn=True)                # [D, F]
        dx = gemm(dgu, w_gate_up, b_mn=True).reshape(ctx.xshape)    # [M, D]
        dw_gate_up = gemm(dgu, x2, a_mn=True, b_mn=True)            # [2F, D]
        return dx, dw_gate_up, dw_down, None


def glu_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, act: str = "silu") -> torch.Tensor:
    return _GluFFN.apply(x, w_gate_up, w_down, act)
