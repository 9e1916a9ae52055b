"""Host runtime pieces that need no GPU: planner layout / chooser / archives, stats block + meshctl, host words,
epoch staleness, the engine-bridge shaped C ABI."""
import ctypes
import json
import os
import subprocess
import sys
import time

import pytest
import torch.distributed as dist

from mesh_b200.runtime import plan, service
from mesh_b200.runtime.rendezvous import ECANCELED, ETIMEDOUT, MeshStale, Rendezvous


def test_planner_layout_chooser_archive(tmp_path):
    offs, one = plan.layout([(0, 3, 1000), (4, 6, 1000), (2, 5, 500)], copies=2, align=256)
    assert offs[0][0] == offs[0][1]                     # disjoint lifetimes share memory
    assert offs[1][0] == offs[0][0] + one               # second copy is the first shifted by one copy
    assert one < 1024 + 1024 + 512
    small, _ = plan.choose_allreduce(4096, 8)
    big, _ = plan.choose_allreduce(256 << 20, 8)
    assert small == "one_shot" and big == "two_shot"
    assert plan.choose_allreduce(256 << 20, 8, nvls=True)[0] == "nvls"
    words = [1, 2, 3, 2 ** 63]
    plan.save(tmp_path / "p.plan", 7, words)
    assert plan.load(tmp_path / "p.plan") == (7, words)
    raw = bytearray((tmp_path / "p.plan").read_bytes())
    raw[-1] ^= 1
    (tmp_path / "bad.plan").write_bytes(raw)
    with pytest.raises(OSError, match="checksum"):
        plan.load(tmp_path / "bad.plan")


def test_stats_block_and_meshctl():
    group = f"t{os.getpid()}"
    assert service.start(group, 0, 1, heartbeat_s=0.05) is False
    try:
        service.count("launches", 5)
        service.count("bytes", 1000, peer=3)
        service.channel(3, "CONNECTED")
        time.sleep(0.12)
        s = service.read(group, 0)
        assert s["alive"] and s["launches"] == 5 and s["bytes_to_peer"][3] == 1000 and s["channels"][3] == "CONNECTED"
        out = subprocess.run([sys.executable, "-m", "mesh_b200.tools.meshctl", "status", "--group", group, "--world", "1", "--ready"],
                             capture_output=True, text=True, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        assert out.returncode == 0 and json.loads(out.stdout)["ranks"][0]["pid"] == os.getpid()
        top = subprocess.run([sys.executable, "-m", "mesh_b200.tools.meshctl", "top", "--group", group, "--world", "4",
                              "--count", "2", "--interval", "0.1"], capture_output=True, text=True,
                             cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        assert top.returncode == 0 and "links (MB/s" in top.stdout and "CONN" in top.stdout and "(no stats block)" in top.stdout
        assert "ranks 1/4 alive" in top.stdout
        service.deadline(0.05)                            # the service thread raises abort once the deadline passes
        time.sleep(0.2)
        assert service.aborted()
    finally:
        service.stop(unlink=True)
    assert service.read(group, 0) is None


def test_host_word_and_epoch():
    w = plan.HostWord()
    w.publish(3)
    w.publish(2)                                          # never moves backwards
    assert w.arrived(3) and not w.arrived(4)
    assert not w.sent(1)
    w.mark_sent(2)
    w.mark_sent(1)
    assert w.sent(2) and not w.sent(3)
    assert w.wait(3, 0.1) == 0 and w.wait(4, 0.05) == ETIMEDOUT
    w.cancel()
    assert w.wait(4, 0.05) == ECANCELED
    rdv = Rendezvous(dist.HashStore(), 0, 1)
    p = plan.Plan(rdv, copies=2)
    rdv.advance_epoch()
    with pytest.raises(MeshStale):
        p.start()


def test_engine_bridge_abi():
    from mesh_b200 import _native
    L = _native.lib()
    L.mesh_open.restype = ctypes.c_void_p
    L.mesh_publish.restype = ctypes.c_uint64
    L.mesh_ipc_inbox.restype = ctypes.POINTER(ctypes.c_float)
    L.mesh_ipc_outbox.restype = ctypes.POINTER(ctypes.c_float)
    h = ctypes.c_void_p(L.mesh_open(ctypes.c_uint64(8)))
    src = (ctypes.c_float * 4)(1, 2, 3, 4)
    assert L.mesh_gather(h, src, ctypes.c_uint64(2), ctypes.c_uint64(4)) == 0
    t = L.mesh_publish(h)
    assert L.mesh_poll(h, ctypes.c_uint64(t)) == 0          # non-blocking: not consumed yet
    inbox, outbox = L.mesh_ipc_inbox(h), L.mesh_ipc_outbox(h)
    for i in range(8):
        outbox[i] = inbox[i] * 2
    L.mesh_ipc_complete(h)
    assert L.mesh_poll(h, ctypes.c_uint64(t)) == 1
    dst = (ctypes.c_float * 4)()
    L.mesh_scatter(h, dst, ctypes.c_uint64(2), ctypes.c_uint64(4))
    assert list(dst) == [2, 4, 6, 8]
    assert L.mesh_gather(h, src, ctypes.c_uint64(6), ctypes.c_uint64(4)) == -1
    L.mesh_close(h)


def _job_with_runtime(rank, world, rdv, group):
    import os
    import torch
    import torch.distributed as dist
    os.environ["MESH_GROUP"] = group
    os.environ["MASTER_PORT"] = os.environ["MESH_AUX_PORT"]      # the launcher's own store holds MASTER_PORT
    import importlib
    cfg = importlib.import_module("mesh_b200.config")
    cfg.set_config(cfg.MeshConfig.from_env())
    from mesh_b200.distributed import init, shutdown
    from mesh_b200.runtime import service
    ctx = init(backend="gloo", device="cpu")
    assert ctx.service, "init() starts the runtime service"
    t = torch.ones(4) * (rank + 1)
    dist.all_reduce(t)
    service.count("step", 7)
    rdv.barrier("running")
    # every rank's block is visible to every other process of the node while the job runs
    for r in range(world):
        s = service.read(group, r)
        assert s is not None and s["alive"] and s["rank"] == r and s["world"] == world and not s["abort"]
        assert s["step"] == 7
    rdv.barrier("read")
    shutdown()
    assert service.read(group, rank) is None, "shutdown() removes this rank's block"


def test_init_starts_the_runtime_service_and_shutdown_stops_it():
    import os
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_job_with_runtime, 2, f"t{os.getpid()}", timeout=120.0)


def test_peer_channels_state_machine_queue_and_bounded_flush():
    """Host-memory channels (no CUDA call): transitions in order only, copies served by the proxy thread, a channel
    that is not connected takes no work, flush waits only for channels with outstanding work."""
    import ctypes
    import pytest
    from mesh_b200.runtime.channels import ChannelError, PeerChannels
    ch = PeerChannels(rank=0, world=3, device=-1)
    assert [ch.state(p) for p in range(3)] == ["OPEN"] * 3
    with pytest.raises(ChannelError):
        ch.advance(1, "CONNECTED")                       # OPEN -> CONNECTED skips MAPPED
    src = (ctypes.c_ubyte * 4096)(*([7] * 4096))
    dst = (ctypes.c_ubyte * 4096)()
    with pytest.raises(ChannelError):
        ch.copy(1, ctypes.addressof(dst), ctypes.addressof(src), 4096)   # not connected yet
    ch.connect_all()
    assert ch.state(2) == "CONNECTED"
    tickets = [ch.copy(1, ctypes.addressof(dst) + 1024 * i, ctypes.addressof(src) + 1024 * i, 1024) for i in range(4)]
    assert tickets == sorted(tickets)
    assert ch.flush(2000) == 0
    assert all(ch.done(1, t) for t in tickets) and bytes(dst) == bytes(src)
    assert ch.bytes(1) == 4096 and ch.bytes(2) == 0
    ch.wait_on_stream(1, tickets[-1], 0, 100)            # issued long ago: returns at once
    ch.advance(2, "HALTED")
    with pytest.raises(ChannelError):
        ch.copy(2, ctypes.addressof(dst), ctypes.addressof(src), 16)
    assert ch.close(1000) == 0


def test_transfer_planner_groups_orders_and_accounts():
    """Declared transfers through the native planner: gradient reductions that nobody reads before the end travel as
    one demand up to the bucket size; a transfer somebody waits for is a demand of its own and goes first when both are
    ready (earliest deadline); demands of one axis never overlap and never start before their value exists; the
    summary adds up; every rank computes the same plan (two calls agree)."""
    import random

    from mesh_b200.runtime.plan import plan_transfers
    end = 100
    grads = [{"bytes": 4 << 20, "axis": 0, "verb": "all_reduce", "at": 60 + 5 * i, "read": end, "groupable": True} for i in range(6)]
    act = {"bytes": 8 << 20, "axis": 0, "verb": "all_gather", "at": 62, "read": 64}
    big = {"bytes": 200 << 20, "axis": 1, "verb": "all_reduce", "at": 10, "read": 20}
    rows = grads + [act, big]
    out, summary = plan_transfers(rows, [8, 2], step_us=10.0, alpha_us=5.0, bucket_bytes=16 << 20, staging_bytes=64 << 20)
    again, summary2 = plan_transfers(rows, [8, 2], step_us=10.0, alpha_us=5.0, bucket_bytes=16 << 20, staging_bytes=64 << 20)
    assert out == again and summary == summary2
    # 6 x 4 MiB into 16 MiB buckets: 4 + 2; the activation gather and the other axis' reduction stand alone
    g = [o["demand"] for o in out[:6]]
    assert g[0] == g[1] == g[2] == g[3] != g[4] == g[5]
    assert out[6]["demand"] not in g and out[7]["demand"] not in g and summary["demands"] == 4
    assert out[7]["pieces"] == 4 and out[7]["algo"] in ("two_shot", "one_shot")
    # the activation is needed at step 64 and is there in time; the gradients are exposed only past the end
    assert out[6]["start_us"] >= 63 * 10.0 and out[6]["exposed_us"] == max(0.0, out[6]["end_us"] - 64 * 10.0)
    # no overlap on an axis, release respected
    for ax in (0, 1):
        spans = sorted({(o["start_us"], o["end_us"], o["demand"]) for o, r in zip(out, rows) if r["axis"] == ax})
        for (s0, e0, _), (s1, e1, _) in zip(spans, spans[1:]):
            assert s1 >= e0 - 1e-9
    for o, r in zip(out, rows):
        last = max(rr["at"] for oo, rr in zip(out, rows) if oo["demand"] == o["demand"])
        assert o["start_us"] >= (last + 1) * 10.0 - 1e-9
    spans = {o["demand"]: (o["start_us"], o["end_us"], o["exposed_us"]) for o in out}
    assert abs(summary["link_us"] - sum(e - s for s, e, _ in spans.values())) < 1e-6
    assert abs(summary["exposed_us"] - sum(x for _, _, x in spans.values())) < 1e-6
    assert abs(summary["makespan_us"] - max(e for _, e, _ in spans.values())) < 1e-6
    # random programs: the same invariants
    rng = random.Random(1)
    for _ in range(20):
        rows = []
        for _ in range(rng.randint(1, 12)):
            at = rng.randint(0, 50)
            rows.append({"bytes": rng.randint(1, 40) << 20, "axis": rng.randint(0, 1), "verb": rng.choice(["all_reduce", "all_gather", "reduce_scatter"]),
                         "at": at, "read": at + rng.randint(0, 30), "groupable": rng.random() < 0.5})
        out, summary = plan_transfers(rows, [4, 2], step_us=7.0, bucket_bytes=64 << 20)
        for ax in (0, 1):
            spans = sorted({(o["start_us"], o["end_us"]) for o, r in zip(out, rows) if r["axis"] == ax})
            assert all(b[0] >= a[1] - 1e-9 for a, b in zip(spans, spans[1:]))
        for o, r in zip(out, rows):
            assert o["start_us"] >= (r["at"] + 1) * 7.0 - 1e-9 and o["exposed_us"] >= 0
            members = [rr for oo, rr in zip(out, rows) if oo["demand"] == o["demand"]]
            if len(members) > 1:
                assert all(m["groupable"] and m["verb"] == "all_reduce" and m["axis"] == r["axis"] for m in members)
                assert sum(m["bytes"] for m in members) <= 64 << 20
                assert max(m["at"] for m in members) < min(m["read"] for m in members)
    import pytest
    with pytest.raises(ValueError):
        plan_transfers([{"bytes": 1, "axis": 3, "verb": "all_reduce", "at": 0, "read": 1}], [2])


def test_pipeline_planner_period_latency_and_copies():
    """The native modulo scheduler: the period is the busiest resource or the tightest dependence cycle, whichever is
    longer; copies = executions alive at once; starts respect dependences and never overlap two tasks of one resource
    modulo the period."""
    from mesh_b200.runtime.plan import plan_pipeline
    chain = [(0, 1, 0), (1, 2, 0)]
    r = plan_pipeline([2.0, 3.0, 1.0], [0, 1, 2], chain)                 # three stages, three resources
    assert abs(r["period"] - 3.0) < 1e-6 and abs(r["latency"] - 6.0) < 1e-6 and r["copies"] == 2
    assert r["starts"] == [0.0, 2.0, 5.0]
    r = plan_pipeline([2.0, 3.0, 1.0], [0, 0, 0], chain)                 # one resource: no overlap possible
    assert abs(r["period"] - 6.0) < 1e-6 and r["copies"] == 1
    r = plan_pipeline([2.0, 3.0, 1.0], [0, 1, 2], chain + [(2, 0, 1)])   # the next execution waits for this one's end
    assert abs(r["period"] - 6.0) < 1e-6 and abs(r["recurrence_bound"] - 6.0) < 1e-6 and r["copies"] == 1
    r = plan_pipeline([2.0, 3.0, 1.0], [0, 1, 2], chain + [(2, 0, 2)])   # ... for the one before: two in flight
    assert abs(r["period"] - 3.0) < 1e-6 and r["copies"] == 2
    # a random instance: check the schedule itself
    import random
    rng = random.Random(5)
    n = 24
    dur = [rng.choice([0.5, 1.0, 2.0, 3.5]) for _ in range(n)]
    res = [rng.randrange(3) for _ in range(n)]
    edges = [(a, b, 0) for b in range(n) for a in range(b) if rng.random() < 0.12] + [(n - 1, 0, 3), (10, 4, 1)]
    r = plan_pipeline(dur, res, edges)
    P, st = r["period"], r["starts"]
    assert P >= max(r["resource_bound"], r["recurrence_bound"]) - 1e-6
    for a, b, lag in edges:
        assert st[b] + lag * P >= st[a] + dur[a] - 1e-6
    for k in range(3):
        spans = sorted((st[i] % P, dur[i]) for i in range(n) if res[i] == k)
        wrapped = [(s, d) for s, d in spans] + [(s + P, d) for s, d in spans]
        for (s0, d0), (s1, _d1) in zip(wrapped, wrapped[1:]):
            assert s1 >= s0 + d0 - 1e-6
    assert r["copies"] == max(1, -(-int(r["latency"] / P * 1e6) // 10 ** 6))
    with pytest.raises(ValueError):
        plan_pipeline([1.0, 1.0], [0, 0], [(0, 1, 0), (1, 0, 0)])        # a cycle within one execution
