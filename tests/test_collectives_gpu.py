"""Collective kernels over the symmetric heap vs. locally computed expectations (every rank builds
all ranks' inputs from seeds), through the ``mesh`` torch.distributed backend and the Communicator."""
import os

import pytest
import torch
import torch.distributed as dist

pytestmark = pytest.mark.gpu


def _inputs(world, n, dtype, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if dtype in (torch.int32, torch.int64):
        return [torch.randint(-50, 50, (n,), generator=g, dtype=dtype) for _ in range(world)]
    return [torch.randn(n, generator=g).to(dtype) for _ in range(world)]


def _run(rank, world, rdv):
    import mesh_b200.distributed.process_group  # noqa: F401
    from mesh_b200.utils.status import check_status
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("mesh", rank=rank, world_size=world,
                            init_method=f"tcp://127.0.0.1:{os.environ['MESH_AUX_PORT']}")
    try:
        for dtype, n in [(torch.float32, 1000), (torch.bfloat16, 4099), (torch.float16, 64), (torch.int32, 33),
                         (torch.float32, 1 << 20), (torch.bfloat16, (3 << 20) + 8), (torch.int64, 7)]:
            ins = _inputs(world, n, dtype, seed=n)
            t = ins[rank].to(dev)
            dist.all_reduce(t)
            if dtype in (torch.bfloat16, torch.float16):
                want = torch.stack([x.float() for x in ins]).sum(0)
                torch.testing.assert_close(t.float().cpu(), want, atol=0.08 * world, rtol=2e-2)
            elif dtype == torch.float32:
                torch.testing.assert_close(t.cpu(), torch.stack(ins).sum(0), atol=1e-4, rtol=1e-5)
            else:
                assert torch.equal(t.cpu(), torch.stack(ins).sum(0))
            # every rank must hold bit-identical results (fixed reduction order)
            both = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(both, t)
            assert all(torch.equal(b, both[0]) for b in both)
            t = ins[rank].to(dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            assert torch.equal(t.cpu(), torch.stack(ins).max(0).values)
        # all_gather_into_tensor / reduce_scatter_tensor / all_to_all_single / broadcast / reduce / p2p
        n = 1536
        ins = _inputs(world, n * world, torch.float32, seed=5)
        out = torch.empty(n * world, device=dev)
        dist.all_gather_into_tensor(out, ins[rank][:n].to(dev))
        assert torch.equal(out.cpu(), torch.cat([x[:n] for x in ins]))
        rs = torch.empty(n, device=dev)
        dist.reduce_scatter_tensor(rs, ins[rank].to(dev))
        torch.testing.assert_close(rs.cpu(), torch.stack(ins).sum(0)[rank * n:(rank + 1) * n], atol=1e-4, rtol=1e-5)
        a2a = torch.empty(n * world, device=dev)
        dist.all_to_all_single(a2a, ins[rank].to(dev))
        assert torch.equal(a2a.cpu(), torch.cat([x[rank * n:(rank + 1) * n] for x in ins]))
        # uneven all-to-all: rank r sends (j + 1) rows of 4 to rank j
        rows_in = [j + 1 for j in range(world)]
        src = torch.arange(sum(rows_in) * 4, dtype=torch.float32).reshape(-1, 4) + 1000 * rank
        dst = torch.empty(((rank + 1) * world, 4), device=dev)
        dist.all_to_all_single(dst, src.to(dev), output_split_sizes=[rank + 1] * world, input_split_sizes=rows_in)
        off = sum(rows_in[:rank])
        want = torch.cat([(torch.arange(sum(rows_in) * 4, dtype=torch.float32).reshape(-1, 4) + 1000 * r)[off:off + rank + 1]
                          for r in range(world)])
        assert torch.equal(dst.cpu(), want)
        b = ins[rank][:100].to(dev)
        dist.broadcast(b, src=world - 1)
        assert torch.equal(b.cpu(), ins[world - 1][:100])
        r = ins[rank].to(dev)
        dist.reduce(r, dst=0)
        if rank == 0:
            torch.testing.assert_close(r.cpu(), torch.stack(ins).sum(0), atol=1e-4, rtol=1e-5)
        comm = dist.group.WORLD._gpu() if hasattr(dist.group.WORLD, "_gpu") else None
        if world > 1:
            nxt, prv = (rank + 1) % world, (rank - 1) % world
            big = ins[rank].repeat(3000)[: (5 << 20)].to(dev)            # 20 MB: several slot-sized pieces
            got = torch.empty_like(big)
            from mesh_b200.distributed import process_group as pgm
            if comm is not None:
                comm.permute(got, big, [(r_, (r_ + 1) % world) for r_ in range(world)])
                assert torch.equal(got.cpu(), ins[prv].repeat(3000)[: (5 << 20)])
            if rank == 0:
                dist.send(ins[0][:77].to(dev), dst=1)
            elif rank == 1:
                x = torch.empty(77, device=dev)
                dist.recv(x, src=0)
                assert torch.equal(x.cpu(), ins[0][:77])
        if world > 1 and comm is not None:
            # Staging alternates call by call: a run of broadcasts from one root must not overwrite a piece that a
            # slow reader has not pulled yet.  Small staging so that one tensor takes many pieces; the last rank
            # starts late (host sleep before its launches) and every broadcast carries different data.
            import time
            from mesh_b200.distributed.comm import Communicator
            mark = comm.heap.mark()
            small = Communicator(comm.heap, staging_bytes=1 << 20, p2p_slot_bytes=1 << 20)
            torch.cuda.synchronize()
            for rep in range(3):
                if rank == world - 1:
                    time.sleep(0.2)
                for j in range(5):
                    want = (torch.arange(3 << 18, dtype=torch.float32) * (j + 1) + rep).to(dev)     # 3 MiB: 3 pieces
                    t = want.clone() if rank == 0 else torch.zeros_like(want)
                    small.broadcast(t, 0)
                    assert torch.equal(t, want), (rep, j)
                x = ins[rank][:4096].to(dev)
                small.reduce(x, 0)
                y = ins[rank][:4096].to(dev) * 2
                small.reduce(y, 0)
                z = ins[rank][:4096].to(dev) * 3
                small.reduce(z, 0)
                if rank == 0:
                    tot = torch.stack(ins).sum(0)[:4096]
                    for got, f in ((x, 1), (y, 2), (z, 3)):
                        torch.testing.assert_close(got.cpu(), tot * f, atol=1e-3, rtol=1e-5)
            # released signal words are handed out again: their new owner must find them at zero, or its first waits
            # pass before the peers have published (the late rank makes that visible as a wrong sum)
            comm.heap.release(mark)
            again = Communicator(comm.heap, staging_bytes=1 << 20, p2p_slot_bytes=1 << 20)
            for rep in range(3):
                if rank == world - 1:
                    time.sleep(0.1)
                v = ins[rank][:2048].to(dev) + rep
                again.all_reduce(v)
                torch.testing.assert_close(v.cpu(), torch.stack(ins).sum(0)[:2048] + rep * world, atol=1e-3, rtol=1e-5)
        dist.barrier()
        check_status()
    finally:
        dist.destroy_process_group()


def test_collectives_world1():
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_run, 1, use_cuda=True, timeout=300.0)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_collectives_multi(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_run, world, use_cuda=True, timeout=300.0)


def test_bounded_wait_reports_timeout():
    """A wait on a word nobody writes runs out after its (short) limit, the kernel returns, the
    status block says TIMEOUT and the context stays usable."""
    import ctypes
    from mesh_b200 import _native
    from mesh_b200.utils.status import MeshTimeout, check_status, status_block
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = status_block()
    rc = _native.lib().mesh_wait_flag_test(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint32(1),
                                           ctypes.c_uint64(50_000_000), ctypes.c_void_p(st.data_ptr()),
                                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    with pytest.raises(MeshTimeout) as e:
        check_status()
    assert e.value.record["site"] == "host_flag" and e.value.record["expected"] == 1
    check_status()                                   # cleared; GPU still answers
    assert torch.ones(4, device="cuda").sum().item() == 4.0
