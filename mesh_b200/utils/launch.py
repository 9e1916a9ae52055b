"""Spawn helpers: run ``fn(rank, world, rendezvous, *args)`` in ``world`` child processes.

Used by the multi-GPU tests and examples; the CPU tests use the same helper with gloo ranks, which
is this package's "fake cluster" (the reference has none and only runs on its live pair).
"""
from __future__ import annotations

import os
import socket
import traceback
from datetime import timedelta


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def free_ports(n: int) -> list[int]:
    """``n`` distinct free ports, found by holding ``n`` bound sockets at once (a port number derived by
    arithmetic from another one is not reserved and may be in use)."""
    socks = []
    try:
        for _ in range(n):
            s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            s.bind(("127.0.0.1", 0))
            socks.append(s)
        return [s.getsockname()[1] for s in socks]
    finally:
        for s in socks:
            s.close()


def _exit_barrier(store, rank: int, world: int, timeout_s: float = 120.0) -> None:
    """Every rank says that it is through; a rank that failed publishes ``spawn-poison`` instead, and the ranks that
    wait here leave at once with an error rather than after the full timeout."""
    import time
    store.set(f"spawn-exit/{rank}", b"1")
    keys = [f"spawn-exit/{r}" for r in range(world)]
    deadline = time.monotonic() + timeout_s
    while True:
        if store.check(keys):
            return
        if store.check(["spawn-poison"]):
            raise RuntimeError(f"rank {rank}: another rank failed ({store.get('spawn-poison').decode(errors='replace')})")
        if time.monotonic() > deadline:
            raise TimeoutError(f"rank {rank}: not every rank reached the end within {timeout_s}s")
        time.sleep(0.005)


def _child(rank: int, world: int, port: int, aux_port: int, fn, args, use_cuda: bool, init_pg: str | None):
    import torch
    import torch.distributed as dist
    from ..runtime.rendezvous import Rendezvous
    watchdog = float(os.environ.get("MESH_SPAWN_WATCHDOG_S", "0") or 0)
    if watchdog > 0:
        # a rank that is still running after this long prints where it is (all threads) and carries on
        import faulthandler
        faulthandler.dump_traceback_later(watchdog, exit=False)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), MESH_AUX_PORT=str(aux_port))
    if use_cuda:
        torch.cuda.set_device(rank)
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=120),
                          wait_for_workers=False)
    if init_pg:
        dist.init_process_group(init_pg, store=dist.PrefixStore("pg", store), rank=rank, world_size=world,
                                timeout=timedelta(seconds=120))
    rdv = Rendezvous(dist.PrefixStore("rdv", store), rank, world, timeout_s=120.0)
    try:
        fn(rank, world, rdv, *args)
        _exit_barrier(store, rank, world)
        # Rank 0's process hosts the store.  It may leave the barrier first, and a store that goes away while another
        # rank is still reading the barrier's keys looks to that rank like a peer that never arrived: so the host
        # stays until every other rank has said that it is through.
        if rank != 0:
            store.set(f"spawn-bye/{rank}", b"1")
        elif world > 1:
            store.wait([f"spawn-bye/{r}" for r in range(1, world)], timedelta(seconds=120))
    except BaseException as e:
        traceback.print_exc()
        try:
            store.set("spawn-poison", f"rank {rank}: {type(e).__name__}".encode())
        except Exception:
            pass
        raise
    finally:
        if init_pg and dist.is_initialized():
            dist.destroy_process_group()


def spawn_ranks(fn, world: int, *args, use_cuda: bool = False, init_pg: str | None = None, timeout: float = 600.0):
    """Run ``fn`` on ``world`` ranks and raise if any child fails.  ``fn`` must be importable."""
    import torch.multiprocessing as mp
    port, aux_port = free_ports(2)
    ctx = mp.start_processes(_child, args=(world, port, aux_port, fn, args, use_cuda, init_pg), nprocs=world, join=False,
                             start_method="spawn")
    import time
    deadline = time.monotonic() + timeout
    while not ctx.join(timeout=1.0):
        if time.monotonic() > deadline:
            for p in ctx.processes:
                if p.is_alive():
                    p.terminate()
            raise TimeoutError(f"spawn_ranks: children did not finish within {timeout}s")
