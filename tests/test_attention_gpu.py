"""tcgen05 flash attention forward vs an fp32 PyTorch statement: causal, sliding window, GQA, head dims, offsets/strides."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(got, want, tol=2e-2):
    err = (got.float() - want.float()).abs().max().item()
    ref = want.float().abs().max().item() + 1e-6
    assert err / ref < tol, f"max err {err} vs {ref}"


@pytest.mark.parametrize("hd,H,Hkv", [(128, 4, 4), (256, 8, 2), (64, 2, 1)])
@pytest.mark.parametrize("Tq,Tk,causal,window", [(256, 256, True, 0), (384, 384, True, 100), (200, 330, False, 0), (512, 512, True, 512)])
def test_flash_forward(hd, H, Hkv, Tq, Tk, causal, window):
    from mesh_b200.ops.attention import attention_ref, flash_attention
    from mesh_b200.utils.status import check_status
    B = 2
    q = torch.randn(B, Tq, H, hd, device="cuda").bfloat16()
    k = torch.randn(B, Tk, Hkv, hd, device="cuda").bfloat16()
    v = torch.randn(B, Tk, Hkv, hd, device="cuda").bfloat16()
    out, lse = flash_attention(q, k, v, causal=causal, window=window, need_lse=True)
    check_status()
    ref, lse_ref = attention_ref(q, k, v, causal, window)
    _close(out, ref)
    torch.testing.assert_close(lse, lse_ref, atol=2e-2, rtol=2e-2)


def test_flash_fused_qkv_view_and_striped_positions():
    from mesh_b200.ops.attention import attention_ref, flash_attention, merge_partials
    B, T, H, Hkv, hd = 1, 256, 4, 2, 128
    qkv = torch.randn(B, T, (H + 2 * Hkv) * hd, device="cuda").bfloat16()
    q = qkv[..., :H * hd].view(B, T, H, hd)
    k = qkv[..., H * hd:(H + Hkv) * hd].view(B, T, Hkv, hd)
    v = qkv[..., (H + Hkv) * hd:].view(B, T, Hkv, hd)
    out = flash_attention(q, k, v, causal=True)
    _close(out, attention_ref(q, k, v, True)[0])
    # two striped halves of the keys merged by log-sum-exp equal attention over all keys
    o_full, _ = attention_ref(q, k, v, True)
    parts = []
    for r in range(2):
        parts.append(flash_attention(q, k[:, r::2].contiguous(), v[:, r::2].contiguous(), causal=True, k_off=r, k_stride=2, need_lse=True))
    o, _ = merge_partials(parts[0][0], parts[0][1], parts[1][0], parts[1][1])
    _close(o, o_full)


def _ring_rank(rank, world, rdv, striped, overlap=False):
    from mesh_b200.config import MeshConfig, set_config
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.ops.attention import attention_ref, ring_attention
    from mesh_b200.utils.status import check_status
    torch.cuda.set_device(rank)
    set_config(MeshConfig.from_env(heap_bytes=512 << 20))
    ctx = MeshContext(rank, world, torch.device("cuda", rank), rdv, None)
    B, T, H, hd = 1, 256 * world, 4, 128
    g = torch.Generator(device="cpu").manual_seed(0)
    q, k, v = (torch.randn(B, T, H, hd, generator=g).bfloat16().cuda() for _ in range(3))
    sl = slice(rank, T, world) if striped else slice(rank * (T // world), (rank + 1) * (T // world))
    o, _ = ring_attention(q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous(), ctx.comm, causal=True,
                          striped=striped, overlap=overlap)
    torch.cuda.synchronize()
    check_status()
    ref, _ = attention_ref(q, k, v, True)
    _close(o, ref[:, sl])
    rdv.barrier("ring-done")
    ctx.heap.close()


@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("striped", [False, True])
def test_ring_attention_two_ranks(striped, overlap):
    """``overlap``: the next KV chunk travels on a side stream under the attention of the current one."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_ring_rank, 2, striped, overlap, use_cuda=True, timeout=300.0)


def _ref_grads(q, k, v, dout, causal, window):
    from mesh_b200.ops.attention import attention_ref
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    o, _ = attention_ref(qf, kf, vf, causal, window)
    o.backward(dout.float())
    return qf.grad, kf.grad, vf.grad


@pytest.mark.parametrize("hd,H,Hkv", [(128, 4, 4), (128, 4, 2), (64, 2, 1), (256, 4, 2)])
@pytest.mark.parametrize("T,causal,window", [(256, True, 0), (384, True, 100), (200, False, 0)])
def test_flash_backward(hd, H, Hkv, T, causal, window):
    """Head size 256 has the forward kernel and a backward in blocks of tensor operations; 64 and 128 both kernels."""
    from mesh_b200.ops.attention import attention
    from mesh_b200.utils.status import check_status
    torch.manual_seed(1)
    B = 2
    q = torch.randn(B, T, H, hd, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(B, T, Hkv, hd, device="cuda").bfloat16().requires_grad_(True)
    v = torch.randn(B, T, Hkv, hd, device="cuda").bfloat16().requires_grad_(True)
    dout = torch.randn(B, T, H, hd, device="cuda").bfloat16()
    out = attention(q, k, v, causal=causal, window=window)
    out.backward(dout)
    torch.cuda.synchronize()
    check_status()
    dq, dk, dv = _ref_grads(q.detach(), k.detach(), v.detach(), dout, causal, window)
    _close(q.grad, dq, 3e-2)
    _close(k.grad, dk, 3e-2)
    _close(v.grad, dv, 3e-2)


def _ring_bwd_rank(rank, world, rdv, striped):
    from mesh_b200.config import MeshConfig, set_config
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.ops.attention import ring_attention_autograd
    from mesh_b200.utils.status import check_status
    torch.cuda.set_device(rank)
    set_config(MeshConfig.from_env(heap_bytes=512 << 20))
    ctx = MeshContext(rank, world, torch.device("cuda", rank), rdv, None)
    B, T, H, Hkv, hd = 1, 256 * world, 4, 2, 128
    g = torch.Generator(device="cpu").manual_seed(0)
    q = torch.randn(B, T, H, hd, generator=g).bfloat16().cuda()
    k, v = (torch.randn(B, T, Hkv, hd, generator=g).bfloat16().cuda() for _ in range(2))
    dout = torch.randn(B, T, H, hd, generator=g).bfloat16().cuda()
    sl = slice(rank, T, world) if striped else slice(rank * (T // world), (rank + 1) * (T // world))
    ql, kl, vl = (t[:, sl].contiguous().requires_grad_(True) for t in (q, k, v))
    o = ring_attention_autograd(ql, kl, vl, ctx.comm, causal=True, striped=striped)
    o.backward(dout[:, sl].contiguous())
    torch.cuda.synchronize()
    check_status()
    dq, dk, dv = _ref_grads(q, k, v, dout, True, 0)
    _close(ql.grad, dq[:, sl], 3e-2)
    _close(kl.grad, dk[:, sl], 3e-2)
    _close(vl.grad, dv[:, sl], 3e-2)
    rdv.barrier("ring-bwd-done")
    ctx.heap.close()


@pytest.mark.parametrize("striped", [False, True])
def test_ring_attention_backward_two_ranks(striped):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_ring_bwd_rank, 2, striped, use_cuda=True, timeout=300.0)


def _ulysses_rank(rank, world, rdv):
    from mesh_b200.config import MeshConfig, set_config
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.ops.attention import ulysses_attention
    from mesh_b200.parallel.topology import AxisContext
    from mesh_b200.utils.status import check_status
    torch.cuda.set_device(rank)
    set_config(MeshConfig.from_env(heap_bytes=512 << 20))
    ctx = MeshContext(rank, world, torch.device("cuda", rank), rdv, None)
    axis = AxisContext("cp", rank, list(range(world)), ctx.device, None, ctx.heap)
    B, T, H, Hkv, hd = 1, 256 * world, 4, 2, 128
    g = torch.Generator(device="cpu").manual_seed(0)
    q = torch.randn(B, T, H, hd, generator=g).bfloat16().cuda()
    k, v = (torch.randn(B, T, Hkv, hd, generator=g).bfloat16().cuda() for _ in range(2))
    dout = torch.randn(B, T, H, hd, generator=g).bfloat16().cuda()
    sl = slice(rank * (T // world), (rank + 1) * (T // world))
    ql, kl, vl = (t[:, sl].contiguous().requires_grad_(True) for t in (q, k, v))
    o = ulysses_attention(ql, kl, vl, axis, causal=True)
    o.backward(dout[:, sl].contiguous())
    torch.cuda.synchronize()
    check_status()
    dq, dk, dv = _ref_grads(q, k, v, dout, True, 0)
    from mesh_b200.ops.attention import attention_ref
    ref, _ = attention_ref(q, k, v, True)
    _close(o, ref[:, sl])
    _close(ql.grad, dq[:, sl], 3e-2)
    _close(kl.grad, dk[:, sl], 3e-2)
    _close(vl.grad, dv[:, sl], 3e-2)
    rdv.barrier("ulysses-done")
    ctx.heap.close()


def test_head_exchange_attention_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_ulysses_rank, 2, use_cuda=True, timeout=300.0)


@pytest.mark.parametrize("hd,H,Hkv,T,causal", [(128, 4, 2, 256, True), (64, 2, 2, 200, False), (256, 2, 1, 256, True)])
def test_flash_forward_with_dropout_matches_the_logical_mask(hd, H, Hkv, T, causal):
    """Dropout inside the kernel: Philox keyed by (head, query position, key position), against the fp32 statement
    that applies the same mask; the kept fraction is 1 - p."""
    from mesh_b200.ops.attention import attention_ref, flash_attention
    from mesh_b200.ops.philox import attention_keep_mask
    from mesh_b200.utils.status import check_status
    torch.manual_seed(3)
    B = 2
    q = torch.randn(B, T, H, hd, device="cuda").bfloat16()
    k = torch.randn(B, T, Hkv, hd, device="cuda").bfloat16()
    v = torch.randn(B, T, Hkv, hd, device="cuda").bfloat16()
    drop = dict(p=0.25, seed=0x1234_5678_9ABC, site=3, execution=7)
    out = flash_attention(q, k, v, causal=causal, dropout=drop)
    check_status()
    ref, _ = attention_ref(q, k, v, causal, dropout=drop)
    _close(out, ref, 3e-2)
    plain, _ = attention_ref(q, k, v, causal)
    assert (out.float() - plain).abs().max() > 0.05                  # the mask did something
    keep = attention_keep_mask(torch.zeros(1, 1, dtype=torch.int64), torch.arange(512)[:, None], torch.arange(512)[None, :],
                               0.25, drop["seed"], drop["site"], drop["execution"])
    assert abs(float(keep.float().mean()) - 0.75) < 0.01


def test_dropout_is_the_same_for_a_shard_of_the_queries_and_of_the_heads():
    from mesh_b200.ops.attention import flash_attention
    torch.manual_seed(4)
    B, T, H, hd = 1, 512, 4, 128
    q, k, v = (torch.randn(B, T, H, hd, device="cuda").bfloat16() for _ in range(3))
    drop = dict(p=0.3, seed=99)
    whole = flash_attention(q, k, v, causal=True, dropout=drop)
    # the second half of the queries, as a sequence shard would hold them (logical positions through q_off)
    part = flash_attention(q[:, 256:].contiguous(), k, v, causal=True, q_off=256, dropout=drop)
    _close(part, whole[:, 256:], 1e-2)                                 # another mask would differ by O(1)
    # heads 2..3 only, as a tensor-parallel rank would hold them
    heads = flash_attention(q[:, :, 2:].contiguous(), k[:, :, 2:].contiguous(), v[:, :, 2:].contiguous(), causal=True,
                            dropout=dict(drop, head_off=2, heads_total=4))
    _close(heads, whole[:, :, 2:], 1e-2)


@pytest.mark.parametrize("hd,H,Hkv", [(128, 4, 2), (64, 2, 2)])
def test_flash_backward_with_dropout(hd, H, Hkv):
    from mesh_b200.ops.attention import attention, attention_ref
    from mesh_b200.utils.status import check_status
    torch.manual_seed(5)
    B, T = 2, 256
    q = torch.randn(B, T, H, hd, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(B, T, Hkv, hd, device="cuda").bfloat16().requires_grad_(True)
    v = torch.randn(B, T, Hkv, hd, device="cuda").bfloat16().requires_grad_(True)
    dout = torch.randn(B, T, H, hd, device="cuda").bfloat16()
    drop = dict(p=0.2, seed=77, site=1)
    attention(q, k, v, causal=True, dropout=drop).backward(dout)
    check_status()
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    o, _ = attention_ref(qf, kf, vf, True, dropout=drop)
    o.backward(dout.float())
    _close(q.grad, qf.grad, 3e-2)
    _close(k.grad, kf.grad, 3e-2)
    _close(v.grad, vf.grad, 3e-2)
