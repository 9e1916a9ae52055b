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


def _ring_rank(rank, world, rdv, striped):
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
    o, _ = ring_attention(q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous(), ctx.comm, causal=True, striped=striped)
    check_status()
    ref, _ = attention_ref(q, k, v, True)
    _close(o, ref[:, sl])
    rdv.barrier("ring-done")
    ctx.heap.close()


@pytest.mark.parametrize("striped", [False, True])
def test_ring_attention_two_ranks(striped):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_ring_rank, 2, striped, use_cuda=True)
