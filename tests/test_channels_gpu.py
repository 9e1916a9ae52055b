"""Peer channels on GPUs: copy-engine transfers served by the proxy thread, ordered after a stream, into a peer's
copy of a symmetric buffer."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_device_channel_copies_in_order_after_a_stream():
    from mesh_b200.runtime.channels import PeerChannels
    ch = PeerChannels(0, 1, device=torch.cuda.current_device())
    ch.connect_all()
    src = torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")
    dst = torch.zeros_like(src)
    s = torch.cuda.current_stream()
    src.fill_(9)                                             # the copy is ordered after this kernel
    t = ch.copy(0, dst.data_ptr(), src.data_ptr(), src.numel(), s.cuda_stream)
    ch.wait_on_stream(0, t, s.cuda_stream)
    assert int(dst.sum()) == 9 * src.numel()
    assert ch.flush(5000) == 0 and ch.done(0, t) and ch.bytes(0) == src.numel()
    assert ch.close() == 0


def _rank(rank, world, rdv):
    import os
    import torch.distributed as dist
    from mesh_b200.distributed import init, shutdown
    os.environ["MASTER_PORT"] = os.environ["MESH_AUX_PORT"]      # the launcher's own store holds MASTER_PORT
    ctx = init(backend="nccl")
    buf = ctx.heap.alloc((1 << 22,), torch.float32)
    buf.local.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    peer = (rank + 1) % world
    src = torch.full((1 << 22,), float(rank + 1), device=ctx.device)
    t = ctx.bulk_put(buf, peer, src)
    assert ctx.channels.flush(10000) == 0 and ctx.channels.done(peer, t)
    dist.barrier()
    torch.cuda.synchronize()
    assert float(buf.local[0]) == float((rank - 1) % world + 1) and float(buf.local.sum()) == float(((rank - 1) % world + 1) * (1 << 22))
    assert ctx.channels.state(peer) == "CONNECTED"
    shutdown()


def test_bulk_put_into_a_peers_symmetric_buffer():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import os
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_rank, 2, use_cuda=True, timeout=300.0)
