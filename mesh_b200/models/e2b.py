"""E2B-class decoder for inference: tensor-parallel prefill + graph-captured greedy decode.

Architecture (the benchmark's decode config, after the reference's Goal B model,
design/collective-goals.md:46-50, design/e2b-crossover-2026-09-16.md:42-52): 30 layers, d_model 2048,
8 query / 2 KV heads of 256, GeGLU FFN 8192, RMSNorm, RoPE theta 1e6, 4 sliding-window (512) layers per
global layer, vocabulary 262144 with tied embeddings; bf16 weights or 4-bit group-64 codes.

Tensor parallelism follows the reference's decode split: attention by heads, FFN by columns, one
all-reduce per block half, KV heads duplicated when there are more ranks than KV heads ("duplicated
cheap compute is free"), vocabulary-parallel LM head with a MAXLOC exchange of 8 bytes per rank.
A decode step is 5 kernels per layer — [norm+QKV+RoPE+cache], [attention], [o-proj+all-reduce+residual],
[norm+gate/up+GeGLU], [down+all-reduce+residual] — plus LM head and argmax, captured once in a CUDA graph and
replayed: no host round trip between tokens (design/e2b-crossover-2026-09-16.md:73-84).
"""
from __future__ import annotations

import dataclasses
import time

import torch

from ..ops import decode as D
from ..ops.gemm import gemm, glu_fwd
from ..ops.norm import rmsnorm_fwd
from ..ops.rope import rope_, rope_tables


@dataclasses.dataclass
class E2BConfig:
    layers: int = 30
    d_model: int = 2048
    q_heads: int = 8
    kv_heads: int = 2
    head_dim: int = 256
    d_ff: int = 8192
    vocab: int = 262144
    window: int = 512
    local_per_global: int = 4
    theta: float = 1e6
    eps: float = 1e-6
    max_seq: int = 1024
    init_std: float = 0.02

    def is_local(self, layer: int) -> bool:
        return (layer + 1) % (self.local_per_global + 1) != 0


def _rand(shape, std, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


class E2BDecoder:
    """Holds this rank's weight shards, KV caches and workspaces; ``prefill`` then ``decode``."""

    def __init__(self, cfg: E2BConfig, ctx, batch: int, quant: str = "bf16", seed: int = 0):
        self.cfg, self.ctx, self.B, self.quant = cfg, ctx, batch, quant
        self.rank, self.world, dev = ctx.rank, ctx.world, ctx.device
        self.dev = dev
        P, r = self.world, self.rank
        c = cfg
        assert c.q_heads % P == 0 and c.d_ff % P == 0 and c.vocab % P == 0
        self.qh = c.q_heads // P
        group = c.q_heads // c.kv_heads
        # KV heads this rank needs: those of its query heads (duplicated across ranks when P > kv_heads)
        q_lo = r * self.qh
        kv_ids = sorted({(q_lo + i) // group for i in range(self.qh)})
        self.kvh = len(kv_ids)
        self.Fl = c.d_ff // P
        self.Vl = c.vocab // P
        hd, d = c.head_dim, c.d_model
        self.layers = []
        for l in range(c.layers):
            s = seed * 1000003 + l * 101
            wq = _rand((c.q_heads * hd, d), c.init_std, s + 1, dev)[q_lo * hd:(q_lo + self.qh) * hd]
            wk_full = _rand((c.kv_heads * hd, d), c.init_std, s + 2, dev)
            wv_full = _rand((c.kv_heads * hd, d), c.init_std, s + 3, dev)
            wk = torch.cat([wk_full[i * hd:(i + 1) * hd] for i in kv_ids])
            wv = torch.cat([wv_full[i * hd:(i + 1) * hd] for i in kv_ids])
            wqkv = torch.cat([wq, wk, wv]).contiguous()
            wo = _rand((d, c.q_heads * hd), c.init_std, s + 4, dev)[:, q_lo * hd:(q_lo + self.qh) * hd].contiguous()
            wg = _rand((c.d_ff, d), c.init_std, s + 5, dev)[r * self.Fl:(r + 1) * self.Fl]
            wu = _rand((c.d_ff, d), c.init_std, s + 6, dev)[r * self.Fl:(r + 1) * self.Fl]
            wgu = torch.cat([wg, wu]).contiguous()
            wd = _rand((d, c.d_ff), c.init_std, s + 7, dev)[:, r * self.Fl:(r + 1) * self.Fl].contiguous()
            L = dict(n1=torch.ones(d, dtype=torch.bfloat16, device=dev), n2=torch.ones(d, dtype=torch.bfloat16, device=dev),
                     wqkv=wqkv, wo=wo, wgu=wgu, wd=wd)
            if quant in ("w4", "w8"):
                quantize, dequantize = (D.quantize_w4, D.dequantize_w4) if quant == "w4" else (D.quantize_w8, D.dequantize_w8)
                for k in ("wqkv", "wo", "wgu", "wd"):
                    if L[k].shape[1] % 512:                   # the quantised kernels walk K in steps of 512: a shard this
                        continue                              # narrow (wo at TP=8) stays bf16
                    codes, scales = quantize(L[k])
                    L[k + "_q"], L[k + "_s"] = codes, scales
                    L[k] = dequantize(codes, scales)          # prefill GEMMs use the dequantised values (same numbers)
            L["kc"] = torch.zeros((batch, self.kvh, c.max_seq, hd), dtype=torch.bfloat16, device=dev)
            L["vc"] = torch.zeros_like(L["kc"])
            self.layers.append(L)
        # tied embedding: every rank keeps the whole table for lookups; its LM-head shard is a row view
        chunks = []
        for ch in range(8):
            chunks.append(_rand((c.vocab // 8, d), c.init_std, seed * 7919 + 500 + ch, dev))
        self.emb = torch.cat(chunks)
        del chunks
        self.lm_head = self.emb[r * self.Vl:(r + 1) * self.Vl]
        if quant in ("w4", "w8"):
            self.lm_q, self.lm_s = (D.quantize_w4 if quant == "w4" else D.quantize_w8)(self.lm_head)
        self.nf = torch.ones(d, dtype=torch.bfloat16, device=dev)
        self.cos, self.sin = rope_tables(c.max_seq, hd, c.theta, device=dev)
        # decode workspaces
        B = batch
        self.pos = torch.zeros(B, dtype=torch.int32, device=dev)
        self.tok = torch.zeros(B, dtype=torch.int32, device=dev)
        self.step = torch.zeros(2, dtype=torch.int32, device=dev)
        self.x = [torch.zeros((B, d), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.q = torch.zeros((B, self.qh * hd), dtype=torch.bfloat16, device=dev)
        self.att_out = torch.zeros((B, self.qh * hd), dtype=torch.bfloat16, device=dev)
        self.h = torch.zeros((B, self.Fl), dtype=torch.bfloat16, device=dev)
        self.logits = torch.zeros((B, self.Vl), dtype=torch.float32, device=dev)
        self.att = D.DecodeAttention(B, self.qh, self.kvh, hd, splits=16, device=dev)
        self.out_tokens = torch.zeros((c.max_seq, B), dtype=torch.int32, device=dev)
        self.calls_per_step = 2 * c.layers
        if P > 1:
            heap = ctx.heap
            # all-reduce slots: [parity][src rank][d_model * 8] 8-byte words; argmax exchange slots
            self.ar = heap.alloc((2 * P * d * 8 * 2,), torch.int32)
            self.xchg = heap.alloc((2 * P * 8 * 2 * 2,), torch.int32)
            self.ar.local.zero_()
            self.xchg.local.zero_()
            torch.cuda.synchronize()
            ctx.rdv.barrier("e2b-slots")
        self.graph = None

    # ------------------------------------------------------------------ pieces
    def _w(self, L, name):
        if self.quant in ("w4", "w8") and (name + "_q") in L:
            return L[name + "_q"], L[name + "_s"]
        return L[name], None

    def _ar(self, call_index):
        return dict(rank=self.rank, world=self.world, recv_ptrs=self.ar.ptrs(), step=self.step,
                    calls_per_step=self.calls_per_step, call_index=call_index)

    def _decode_step(self):
        """Enqueue one token for every sequence (reads self.tok / self.pos, writes them back)."""
        c = self.cfg
        x, x1 = self.x
        D.decode_embed(self.emb, self.tok, x)
        import os
        # measured on a B200: asking for whole next matrices (tens of MB) while the current one streams halves the
        # decode rate (the lines are evicted again before they are used and cross HBM twice); off unless switched on,
        # and then capped (MESH_DECODE_PREFETCH_MB, default 8 MB: enough to bridge a kernel boundary)
        ahead = os.environ.get("MESH_DECODE_PREFETCH_NEXT", "0") == "1"
        head = self.lm_q if self.quant in ("w4", "w8") else self.lm_head

        def nxt(l, name):
            """Weights of the linear layer that follows (its codes when quantised): prefetched into L2 by this one."""
            if not ahead:
                return None
            if name == "head":
                return head
            return self._w(self.layers[l], name)[0]
        for l, L in enumerate(self.layers):
            w, s = self._w(L, "wqkv")
            D.decode_linear(x, w, scales=s, norm_w=L["n1"], eps=c.eps, mode=D.QKV, next_weights=nxt(l, "wo"),
                            qkv=dict(q_heads=self.qh, kv_heads=self.kvh, head_dim=c.head_dim, pos=self.pos, cos=self.cos,
                                     sin=self.sin, q_out=self.q, k_cache=L["kc"], v_cache=L["vc"], max_seq=c.max_seq))
            self.att(self.q, L["kc"], L["vc"], self.pos, self.att_out, window=c.window if c.is_local(l) else 0)
            w, s = self._w(L, "wo")
            if self.world > 1:
                D.decode_linear(self.att_out, w, scales=s, mode=D.ALLREDUCE, out=x1, residual=x, ar=self._ar(2 * l),
                                next_weights=nxt(l, "wgu"))
            else:
                D.decode_linear(self.att_out, w, scales=s, out=x1, residual=x, next_weights=nxt(l, "wgu"))
            w, s = self._w(L, "wgu")
            D.decode_linear(x1, w, scales=s, norm_w=L["n2"], eps=c.eps, mode=D.GLU, act="gelu_tanh", out=self.h,
                            next_weights=nxt(l, "wd"))
            after = nxt(l + 1, "wqkv") if l + 1 < len(self.layers) else nxt(l, "head")
            w, s = self._w(L, "wd")
            if self.world > 1:
                D.decode_linear(self.h, w, scales=s, mode=D.ALLREDUCE, out=x, residual=x1, ar=self._ar(2 * l + 1),
                                next_weights=after)
            else:
                D.decode_linear(self.h, w, scales=s, out=x, residual=x1, next_weights=after)
        if self.quant in ("w4", "w8"):
            D.decode_linear(x, self.lm_q, scales=self.lm_s, norm_w=self.nf, eps=c.eps, out=self.logits)
        else:
            D.decode_linear(x, self.lm_head, norm_w=self.nf, eps=c.eps, out=self.logits)
        D.decode_argmax(self.logits, self.tok, self.pos, vocab_offset=self.rank * self.Vl, rank=self.rank, world=self.world,
                        xchg_ptrs=self.xchg.ptrs() if self.world > 1 else None, step=self.step)

    def _mm(self, x, L, name):
        """Prefill projection: quantised weights go through the GEMM that dequantises them in registers."""
        if self.quant in ("w4", "w8") and (name + "_q") in L and x.shape[1] % 64 == 0:
            from ..ops.gemm import gemm_q
            return gemm_q(x, L[name + "_q"], L[name + "_s"])
        return gemm(x, L[name])

    # ------------------------------------------------------------------ prefill
    def prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        """prompt int32 [B, T] (same on every rank) -> first generated token [B]; fills the KV caches."""
        c = self.cfg
        B, T = prompt.shape
        hd, d = c.head_dim, c.d_model
        comm = self.ctx.comm if self.world > 1 else None
        x = self.emb[prompt.reshape(-1).long()]                                       # [B*T, d]
        positions = torch.arange(T, dtype=torch.int32, device=self.dev).repeat(B)
        from ..ops.attention import flash_attention
        att_out = torch.empty((B * T, self.qh * hd), dtype=torch.bfloat16, device=self.dev)
        for l, L in enumerate(self.layers):
            h, _, _ = rmsnorm_fwd(x, L["n1"], c.eps)
            qkv = self._mm(h, L, "wqkv")
            qv = qkv[:, :self.qh * hd].view(B * T, self.qh, hd)
            kv = qkv[:, self.qh * hd:(self.qh + self.kvh) * hd].view(B * T, self.kvh, hd)
            rope_(qv, positions, self.cos, self.sin)
            rope_(kv, positions, self.cos, self.sin)
            vv = qkv[:, (self.qh + self.kvh) * hd:].view(B * T, self.kvh, hd)
            L["kc"][:, :, :T].copy_(kv.view(B, T, self.kvh, hd).transpose(1, 2))
            L["vc"][:, :, :T].copy_(vv.view(B, T, self.kvh, hd).transpose(1, 2))
            # prefill attention straight from the fused qkv matrix (tcgen05 flash attention; no copies of q, k, v)
            flash_attention(qv.view(B, T, self.qh, hd), kv.view(B, T, self.kvh, hd), vv.view(B, T, self.kvh, hd), causal=True,
                            window=c.window if c.is_local(l) else 0, out=att_out.view(B, T, self.qh, hd))
            o = self._mm(att_out, L, "wo")
            if comm is not None:
                comm.all_reduce(o)
            x = x + o
            h, _, _ = rmsnorm_fwd(x, L["n2"], c.eps)
            a, _ = glu_fwd(h, L["wgu"], act="gelu_tanh", save_gu=False)
            o = self._mm(a, L, "wd")
            if comm is not None:
                comm.all_reduce(o)
            x = x + o
        last = x.view(B, T, d)[:, -1].contiguous()
        if self.quant in ("w4", "w8"):
            D.decode_linear(last, self.lm_q, scales=self.lm_s, norm_w=self.nf, eps=c.eps, out=self.logits)
        else:
            D.decode_linear(last, self.lm_head, norm_w=self.nf, eps=c.eps, out=self.logits)
        self.pos.fill_(T - 1)
        D.decode_argmax(self.logits, self.tok, self.pos, vocab_offset=self.rank * self.Vl, rank=self.rank, world=self.world,
                        xchg_ptrs=self.xchg.ptrs() if self.world > 1 else None, step=self.step)
        return self.tok.clone()

    # ------------------------------------------------------------------ decode
    def weight_bytes(self) -> int:
        """Bytes of weights (codes and scales when quantised) one decode step reads on this rank."""
        n = 0
        for L in self.layers:
            for k in ("wqkv", "wo", "wgu", "wd"):
                if (k + "_q") in L and self.quant in ("w4", "w8"):
                    n += L[k + "_q"].numel() + L[k + "_s"].numel() * 2
                else:
                    n += L[k].numel() * 2
        if self.quant in ("w4", "w8"):
            n += self.lm_q.numel() + self.lm_s.numel() * 2
        else:
            n += self.lm_head.numel() * 2
        return n

    def step_kernel_fits(self) -> bool:
        """Whether the whole step can run as one cooperative kernel (``ops/decode.py::DecodeStep``)."""
        return self.qh // self.kvh <= 4

    def capture(self, mode: str | None = None):
        """Prepare the decode step for replay.  ``mode``: ``"step"``: the whole step as one cooperative kernel;
        ``"graph"``: the step's launches recorded in a CUDA graph (after a warm-up step on a side stream).
        Default: ``MESH_DECODE_MODE``, else ``"graph"``."""
        import os
        mode = mode or os.environ.get("MESH_DECODE_MODE") or "graph"
        if mode == "step" and not self.step_kernel_fits():
            raise ValueError("the step kernel takes groups of at most 4 query heads per KV head")
        if mode not in ("step", "graph"):
            raise ValueError(f"decode mode {mode!r}: 'step' or 'graph'")
        self.mode = mode
        if mode == "step":
            saved = (self.pos.clone(), self.tok.clone(), self.step.clone())
            with D.record_step(self.dev) as st:
                self._decode_step()
            self.stepk, self.graph = st, None
            return saved
        self.stepk = None
        s = torch.cuda.Stream(device=self.dev)
        s.wait_stream(torch.cuda.current_stream())
        saved = (self.pos.clone(), self.tok.clone(), self.step.clone())
        with torch.cuda.stream(s):
            self._decode_step()              # warm-up: loads kernels, sizes nothing new
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        if self.world > 1:
            self.ctx.rdv.barrier("e2b-warm")
        g = torch.cuda.CUDAGraph()
        # thread_local: the runtime's service threads (status monitor, channel proxy) make CUDA calls on their own
        # streams; with the default, process-wide mode such a call during the capture invalidates it (seen with the
        # longer captures of batch 8)
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            self._decode_step()
        self.graph = g
        return saved

    def decode(self, steps: int, record: bool = True) -> torch.Tensor:
        """Greedy-decode ``steps`` tokens per sequence by replaying the captured step."""
        if self.graph is None and getattr(self, "stepk", None) is None:
            raise RuntimeError("call capture() first")
        for i in range(steps):
            if self.graph is not None:
                self.graph.replay()
            else:
                self.stepk.run()
            if record:
                self.out_tokens[i].copy_(self.tok)
        return self.out_tokens[:steps]


def bench_decode(ctx, steps: int = 256, prompt_len: int = 512, configs=(("bf16", 1), ("bf16", 8), ("w4", 1), ("w4", 8), ("w8", 1), ("w8", 8)),
                 cfg: E2BConfig | None = None, mode: str | None = None) -> dict:
    """Decode tokens/s (whole job: batch * steps / time), device-timed, max over ranks.  ``mode``: how the step is
    replayed (``E2BDecoder.capture``)."""
    import torch.distributed as dist
    cfg = cfg or E2BConfig()
    res = {"model": "E2B-class decoder (30L, d2048, 8q/2kv x256, GeGLU 8192, SWA 512 4:1, vocab 262144 tied)",
           "prompt": prompt_len, "decode_steps": steps, "tp": ctx.world, "runs": []}
    if ctx.world > 1:
        _ = ctx.comm                      # allocated before the mark below, so it outlives the per-run release
    from ..config import capacity
    from ..runtime.monitor import ErrorMonitor
    from ..utils.status import check_status, clear_abort
    for quant, B in configs:
        mark = ctx.heap.mark() if ctx.world > 1 else None
        try:
            m = E2BDecoder(cfg, ctx, B, quant)
        except Exception as e:      # a configuration that cannot be built is reported, the others still run
            res["runs"].append({"weights": quant, "batch": B, "error": f"{type(e).__name__}: {e}"[:200]})
            if mark is not None:
                ctx.heap.release(mark)
            continue
        g = torch.Generator(device="cpu").manual_seed(11)
        prompt = torch.randint(0, cfg.vocab, (B, prompt_len), generator=g, dtype=torch.int32).to(ctx.device)
        m.prefill(prompt)
        torch.cuda.synchronize()
        saved = m.capture(mode)
        # the warm-up and capture advanced nothing visible except pos/tok/step of the warm-up step: restore
        m.pos.copy_(saved[0]); m.tok.copy_(saved[1])
        if ctx.world > 1:
            # step counters must agree across ranks: they do (every rank ran the same two steps)
            dist.barrier()
        torch.cuda.synchronize()
        # If a rank falls out of step, every later kernel of the replayed graph would sit out its full wait limit.
        # A monitor (started after the capture: a second thread may not touch the device while a stream is being
        # captured) spreads the abort flag after the first failure, so the rest of the run drains at once.
        monitor = ErrorMonitor(ctx.device, interval_ms=10)
        try:
            import time as _time
            t_dead = _time.perf_counter() + 1.0
            while monitor.report()["polls"] < 1 and _time.perf_counter() < t_dead:
                _time.sleep(0.002)                   # its set-up (pinned buffer, stream) is over before the timed region
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            m.decode(steps, record=False)
            e1.record()
            torch.cuda.synchronize()
        finally:
            monitor.stop()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], device=ctx.device, dtype=torch.float64)
        if ctx.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        # a run in which any rank timed out or was cancelled is not reported as a number; every rank learns of it,
        # so that all of them leave the loop together
        from ..utils.status import decode, status_block
        torch.cuda.synchronize()
        bad = torch.tensor([int(decode(status_block(ctx.device))["code"] != "OK")], device=ctx.device)
        if ctx.world > 1:
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad):
            clear_abort(ctx.device)
            check_status(ctx.device)
            raise RuntimeError("decode: another rank reported a device-side failure")
        res["runs"].append({"weights": quant, "batch": B, "mode": m.mode, "ms_per_token": round(ms / steps, 4),
                            "tokens_per_s": round(B * steps / (ms * 1e-3), 1), "weight_bytes": m.weight_bytes(),
                            "frac_of_weight_streaming_bound": round(m.weight_bytes() / (capacity().get("hbm_gbs", 6650.0) * 1e9)
                                                                    / (ms / steps * 1e-3), 3)})
        del m
        torch.cuda.empty_cache()
        if mark is not None:
            ctx.heap.release(mark)
    return res
