"""Decode kernels against plain PyTorch fp32 statements of the same ops."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(got, want, tol=2e-2):
    err = (got.float() - want.float()).abs().max().item()
    ref = want.float().abs().max().item() + 1e-6
    assert err / ref < tol, f"max err {err} vs {ref}"


@pytest.mark.parametrize("B", [1, 3, 8])
@pytest.mark.parametrize("N,K", [(2048, 2048), (768, 256), (2048, 1024), (512, 8192)])
def test_decode_linear_store_and_norm(B, N, K):
    from mesh_b200.ops.decode import decode_linear
    from mesh_b200.ops.norm import rmsnorm_ref
    x = torch.randn(B, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    nw = (torch.randn(K, device="cuda") * 0.1 + 1).bfloat16()
    res = torch.randn(B, N, device="cuda").bfloat16()
    y = decode_linear(x, w)
    _close(y, x.float() @ w.float().T)
    y2 = decode_linear(x, w, norm_w=nw, residual=res, out_f32=True)
    _close(y2, rmsnorm_ref(x, nw).float() @ w.float().T + res.float())


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_decode_linear_glu(act):
    from mesh_b200.ops.decode import GLU, decode_linear
    B, K, F = 4, 2048, 1024
    x = torch.randn(B, K, device="cuda").bfloat16()
    w = (torch.randn(2 * F, K, device="cuda") * 0.03).bfloat16()
    y = decode_linear(x, w, mode=GLU, act=act)
    g, u = x.float() @ w[:F].float().T, x.float() @ w[F:].float().T
    a = torch.nn.functional.silu(g) if act == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
    _close(y, a * u)


@pytest.mark.parametrize("B,K,N", [(5, 2048, 1024), (1, 8192, 2048), (8, 512, 64), (3, 1024, 256), (2, 4096, 48)])
def test_decode_linear_w4(B, K, N, monkeypatch):
    """4-bit group-64 weights: the 16-byte-per-lane reader (K slices of 128 and more per warp) and the 4-byte reader
    (narrower slices, or MESH_DECODE_W4_NARROW=1) against the dequantised weights in fp32."""
    from mesh_b200.ops.decode import decode_linear, dequantize_w4, quantize_w4
    x = torch.randn(B, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
    codes, scales = quantize_w4(w)
    wd = dequantize_w4(codes, scales)
    assert (wd.float() - w.float()).abs().max() < 0.02 * 5 / 7 + 1e-3       # half a quantisation step at 5 sigma
    y = decode_linear(x, codes, scales=scales)
    _close(y, x.float() @ wd.float().T)


@pytest.mark.parametrize("B,K,N", [(5, 2048, 1024), (1, 8192, 2048), (8, 512, 64), (3, 1024, 256)])
def test_decode_linear_w8(B, K, N):
    from mesh_b200.ops.decode import decode_linear, dequantize_w8, quantize_w8
    x = torch.randn(B, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
    codes, scales = quantize_w8(w)
    wd = dequantize_w8(codes, scales)
    assert (wd.float() - w.float()).abs().max() < 0.02 * 5 / 127 + 5e-4
    y = decode_linear(x, codes, scales=scales)
    _close(y, x.float() @ wd.float().T)


def test_decode_glu_and_norm_with_quantised_weights():
    from mesh_b200.ops.decode import GLU, decode_linear, dequantize_w4, dequantize_w8, quantize_w4, quantize_w8
    B, K, F = 4, 2048, 512
    x = torch.randn(B, K, device="cuda").bfloat16()
    nw = (torch.randn(K, device="cuda") * 0.1 + 1).bfloat16()
    w = (torch.randn(2 * F, K, device="cuda") * 0.02).bfloat16()
    xn = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()).bfloat16().float()
    for quantize, dequantize in ((quantize_w4, dequantize_w4), (quantize_w8, dequantize_w8)):
        codes, scales = quantize(w)
        wd = dequantize(codes, scales).float()
        y = decode_linear(x, codes, scales=scales, norm_w=nw, eps=1e-6, mode=GLU, act="gelu_tanh")
        g, u = xn @ wd[:F].T, xn @ wd[F:].T
        _close(y, torch.nn.functional.gelu(g, approximate="tanh") * u)


def test_decode_qkv_rope_cache():
    from mesh_b200.ops.decode import QKV, decode_linear
    from mesh_b200.ops.rope import rope_ref, rope_tables
    B, K, qh, kvh, hd, S = 3, 2048, 4, 1, 256, 64
    x = torch.randn(B, K, device="cuda").bfloat16()
    w = (torch.randn((qh + 2 * kvh) * hd, K, device="cuda") * 0.03).bfloat16()
    cos, sin = rope_tables(S, hd, 1e6)
    pos = torch.tensor([5, 0, 63], dtype=torch.int32, device="cuda")
    q = torch.zeros(B, qh * hd, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(B, kvh, S, hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    decode_linear(x, w, mode=QKV, qkv=dict(q_heads=qh, kv_heads=kvh, head_dim=hd, pos=pos, cos=cos, sin=sin, q_out=q,
                                           k_cache=kc, v_cache=vc, max_seq=S))
    y = (x.float() @ w.float().T)
    qr = rope_ref(y[:, :qh * hd].view(B, qh, hd), pos, cos, sin)
    kr = rope_ref(y[:, qh * hd:(qh + kvh) * hd].view(B, kvh, hd), pos, cos, sin)
    vr = y[:, (qh + kvh) * hd:].view(B, kvh, hd)
    _close(q.view(B, qh, hd), qr)
    for b in range(B):
        _close(kc[b, :, pos[b]], kr[b])
        _close(vc[b, :, pos[b]], vr[b])
    assert kc.abs().sum(-1).count_nonzero().item() == B * kvh         # only one position written per sequence


@pytest.mark.parametrize("window", [0, 16])
@pytest.mark.parametrize("T", [1, 7])
def test_decode_attention(window, T):
    from mesh_b200.ops.decode import DecodeAttention
    B, qh, kvh, hd, S = 2, 8, 2, 256, 96
    kc = torch.randn(B, kvh, S, hd, device="cuda").bfloat16()
    vc = torch.randn(B, kvh, S, hd, device="cuda").bfloat16()
    q = torch.randn(B, T, qh, hd, device="cuda").bfloat16()
    pos = torch.tensor([40, 70], dtype=torch.int32, device="cuda")
    att = DecodeAttention(B, qh, kvh, hd, splits=4, tokens_per_seq=T)
    out = torch.empty(B, T, qh * hd, device="cuda", dtype=torch.bfloat16)
    att(q, kc, vc, pos, out, window=window)
    att(q, kc, vc, pos, out, window=window)      # second launch: counters were left at zero
    for b in range(B):
        for t in range(T):
            p = int(pos[b]) + t
            lo = max(0, p - window + 1) if window else 0
            k = kc[b, :, lo:p + 1].float().repeat_interleave(qh // kvh, 0)
            v = vc[b, :, lo:p + 1].float().repeat_interleave(qh // kvh, 0)
            s = torch.einsum("hd,hkd->hk", q[b, t].float(), k) / math.sqrt(hd)
            want = torch.einsum("hk,hkd->hd", torch.softmax(s, -1), v).reshape(-1)
            _close(out[b, t], want)


def test_decode_argmax():
    from mesh_b200.ops.decode import decode_argmax
    logits = torch.randn(4, 50000, device="cuda")
    logits[2, 777] = 50.0
    logits[2, 40000] = 50.0                       # tie: lowest index wins
    tok = torch.zeros(4, dtype=torch.int32, device="cuda")
    pos = torch.zeros(4, dtype=torch.int32, device="cuda")
    step = torch.zeros(2, dtype=torch.int32, device="cuda")
    decode_argmax(logits, tok, pos, vocab_offset=1000, step=step)
    assert tok.tolist() == (logits.argmax(-1) + 1000).tolist() and tok[2].item() == 1777
    assert pos.tolist() == [1, 1, 1, 1] and step.tolist() == [1, 0]
