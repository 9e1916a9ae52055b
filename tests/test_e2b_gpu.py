"""E2B-class decoder: prefill + graph-replayed decode vs a plain PyTorch fp32 model with the same weights;
tensor-parallel vs solo."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _small_cfg(q_heads=4):
    """``q_heads=8`` makes every layer 1024 wide or more: what the one-kernel step needs of 4-bit weights."""
    from mesh_b200.models.e2b import E2BConfig
    return E2BConfig(layers=5, d_model=1024, q_heads=q_heads, kv_heads=2, head_dim=128, d_ff=2048, vocab=4096, window=16,
                     local_per_global=4, max_seq=96, init_std=0.05)


def _ref_logits(m, tokens):
    """fp32 reference of the whole model on a token matrix [B, T] -> logits of the last position."""
    c = m.cfg
    B, T = tokens.shape
    hd = c.head_dim
    x = m.emb[tokens.long()].float()
    cos, sin = m.cos[:T].float(), m.sin[:T].float()
    idx = torch.arange(T, device=x.device)
    for l, L in enumerate(m.layers):
        def norm(v, w):
            return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + c.eps) * w.float()
        h = norm(x, L["n1"])
        qkv = h @ L["wqkv"].float().T
        q = qkv[..., :c.q_heads * hd].view(B, T, c.q_heads, hd)
        k = qkv[..., c.q_heads * hd:(c.q_heads + c.kv_heads) * hd].view(B, T, c.kv_heads, hd)
        v = qkv[..., (c.q_heads + c.kv_heads) * hd:].view(B, T, c.kv_heads, hd)

        def rope(t):
            a, b = t[..., :hd // 2], t[..., hd // 2:]
            cs, sn = cos[None, :, None, :], sin[None, :, None, :]
            return torch.cat([a * cs - b * sn, b * cs + a * sn], -1)
        q, k = rope(q), rope(k)
        g = c.q_heads // c.kv_heads
        k = k.repeat_interleave(g, 2)
        v = v.repeat_interleave(g, 2)
        s = torch.einsum("bthd,bshd->bhts", q, k) / math.sqrt(hd)
        mask = idx[None, :] > idx[:, None]
        if c.is_local(l):
            mask = mask | (idx[None, :] <= idx[:, None] - c.window)
        s = s.masked_fill(mask[None, None], float("-inf"))
        o = torch.einsum("bhts,bshd->bthd", torch.softmax(s, -1), v).reshape(B, T, -1)
        x = x + o @ L["wo"].float().T
        h = norm(x, L["n2"])
        F = c.d_ff
        a = torch.nn.functional.gelu(h @ L["wgu"][:F].float().T, approximate="tanh") * (h @ L["wgu"][F:].float().T)
        x = x + a @ L["wd"].float().T
    xf = x[:, -1]
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + c.eps) * m.nf.float()
    if m.quant in ("w4", "w8"):          # the LM head reads the codes of the tied table
        from mesh_b200.ops.decode import dequantize_w4, dequantize_w8
        return xf @ (dequantize_w4 if m.quant == "w4" else dequantize_w8)(m.lm_q, m.lm_s).float().T
    return xf @ m.emb.float().T


def _solo_ctx():
    import torch.distributed as dist
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.runtime.rendezvous import Rendezvous
    return MeshContext(0, 1, torch.device("cuda", torch.cuda.current_device()), Rendezvous(dist.HashStore(), 0, 1), None)


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


@pytest.mark.parametrize("mode", ["step", "graph"])
@pytest.mark.parametrize("quant", ["bf16", "w4", "w8"])
def test_e2b_solo_matches_reference(quant, mode):
    from mesh_b200.models.e2b import E2BDecoder
    from mesh_b200.utils.status import check_status
    cfg = _small_cfg(8 if mode == "step" else 4)
    B, T, steps = 2, 24, 6
    m = E2BDecoder(cfg, _solo_ctx(), B, quant)
    prompt = torch.randint(0, cfg.vocab, (B, T), dtype=torch.int32, device="cuda")
    m.prefill(prompt)
    assert _rel(m.logits, _ref_logits(m, prompt)) < 0.05
    seq = torch.cat([prompt, m.tok[:, None]], 1)
    m.capture(mode)
    m.pos.fill_(T); m.tok.copy_(seq[:, -1])
    for _ in range(steps):
        m.decode(1)
        ref = _ref_logits(m, seq)
        assert _rel(m.logits, ref) < 0.06
        seq = torch.cat([seq, m.tok[:, None]], 1)        # follow the kernel's own greedy choice
    check_status()
    assert m.pos.tolist() == [T + steps] * B


@pytest.mark.parametrize("quant,B", [("bf16", 1), ("bf16", 8), ("w4", 3), ("w8", 8)])
def test_step_kernel_follows_separate_launches(quant, B):
    """The whole step as one cooperative kernel against the step's separate launches, token after token from the same
    inputs: the layers are the same arithmetic with the sums over k taken in another order, so the logits agree to
    rounding, the chosen tokens wherever the best logit leads by more than that, and the counters exactly."""
    from mesh_b200.models.e2b import E2BDecoder
    from mesh_b200.utils.status import check_status
    cfg = _small_cfg(8)
    T, steps = 20, 10
    prompt = torch.randint(0, cfg.vocab, (B, T), dtype=torch.int32, device="cuda")
    models = []
    for mode in ("graph", "step"):
        m = E2BDecoder(cfg, _solo_ctx(), B, quant)
        first = m.prefill(prompt)
        m.capture(mode)                      # the graph form runs a warm-up step: put the state back
        m.pos.fill_(T - 1); m.tok.copy_(first)
        models.append(m)
    g, s = models
    g0, s0 = int(g.step[0]), int(s.step[0])
    for _ in range(steps):
        s.tok.copy_(g.tok); s.pos.copy_(g.pos)
        g.decode(1); s.decode(1)
        a, b = g.logits.float(), s.logits.float()
        assert float((a - b).square().mean().sqrt() / a.square().mean().sqrt()) < 2e-2
        top = a.topk(2, dim=-1).values
        clear = (top[:, 0] - top[:, 1]) > 0.1 * a.abs().amax(-1)
        assert torch.equal(g.tok[clear], s.tok[clear])
        assert torch.equal(g.pos, s.pos)
    check_status()
    assert int(g.step[0]) - g0 == int(s.step[0]) - s0 == steps
    s.decode(3)                                # several steps back to back: the barrier words carry over
    check_status()
    assert s.pos.tolist() == [T - 1 + steps + 3] * B


def _tp_rank(rank, world, rdv):
    import torch.distributed as dist
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.models.e2b import E2BDecoder
    from mesh_b200.utils.status import check_status
    torch.cuda.set_device(rank)
    from mesh_b200.config import MeshConfig, set_config
    set_config(MeshConfig.from_env(heap_bytes=256 << 20))
    ctx = MeshContext(rank, world, torch.device("cuda", rank), rdv, None)
    cfg = _small_cfg()
    B, T, steps = 2, 24, 5
    g = torch.Generator(device="cpu").manual_seed(3)
    prompt = torch.randint(0, cfg.vocab, (B, T), generator=g, dtype=torch.int32).cuda()
    tp = E2BDecoder(cfg, ctx, B, "bf16")
    solo = E2BDecoder(cfg, _solo_ctx(), B, "bf16")
    t_tp = tp.prefill(prompt)
    ref = _ref_logits(solo, prompt)
    Vl = cfg.vocab // world
    assert _rel(tp.logits, ref[:, rank * Vl:(rank + 1) * Vl]) < 0.05
    seq = torch.cat([prompt, t_tp[:, None]], 1)
    tp.capture()
    tp.pos.fill_(T); tp.tok.copy_(seq[:, -1])
    for _ in range(steps):
        tp.decode(1)
        ref = _ref_logits(solo, seq)
        assert _rel(tp.logits, ref[:, rank * Vl:(rank + 1) * Vl]) < 0.06
        seq = torch.cat([seq, tp.tok[:, None]], 1)
    # every rank chose the same tokens
    mine = seq.clone()
    all_ = rdv.exchange("tokens", mine.cpu().tolist())
    assert all(a == all_[0] for a in all_)
    check_status()
    rdv.barrier("tp-done")
    ctx.heap.close()


@pytest.mark.parametrize("mode", ["graph", "step"])
@pytest.mark.parametrize("world", [2, 4])
def test_e2b_tensor_parallel(world, mode, monkeypatch):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    monkeypatch.setenv("MESH_DECODE_MODE", mode)          # the ranks inherit it
    spawn_ranks(_tp_rank, world, use_cuda=True, timeout=300.0)
