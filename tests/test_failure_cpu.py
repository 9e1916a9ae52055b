"""Host-side failure detection, elastic regroup and supervised restart (CPU / gloo ranks; no GPU is involved)."""
import json
import os
import subprocess
import sys
import textwrap

import pytest
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_rank_leaves_between_steps_survivors_regroup():
    # rank 2 leaves at step 3; ranks 0 and 1 learn of it on the host before their next launch and continue as two
    import torch.multiprocessing as mp
    from mesh_b200.utils.launch import free_port
    port = free_port()
    ctx = mp.start_processes(_child_noexit, args=(3, port), nprocs=3, join=False, start_method="spawn")
    import time
    t0 = time.time()
    while not ctx.join(timeout=1.0):
        assert time.time() - t0 < 120


def _child_noexit(rank, world, port):
    from datetime import timedelta
    from mesh_b200.runtime.failure import FailureDetector, PeerLost
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=60), wait_for_workers=False)
    fd = FailureDetector(store, rank, world, timeout_s=3.0)
    store.add("up", 1)
    import time
    while int(store.add("up", 0)) < world:
        time.sleep(0.01)
    members = list(range(world))
    done_steps = 0
    for step in range(6):
        if rank == 2 and step == 3:
            fd.leave()
            break
        try:
            fd.check(step)
        except PeerLost as e:
            assert e.lost == [2]
            _, new_world, members = fd.regroup(e.lost)
            assert new_world == 2 and fd.epoch == 1
        # the step's synchronisation among the CURRENT members (a counter in the store stands in for a collective)
        key = f"step/{fd.epoch}/{step}"
        store.add(key, 1)
        t0 = time.time()
        while int(store.add(key, 0)) < len(members):
            if time.time() - t0 > 1.0:
                # a member may have left after our check: re-check instead of waiting forever
                try:
                    fd.check(step)
                except PeerLost as e:
                    _, _, members = fd.regroup(e.lost)
                    key = f"step/{fd.epoch}/{step}"
                    store.add(key, 1)
                t0 = time.time()
            time.sleep(0.005)
        done_steps += 1
    if rank != 2:
        assert done_steps == 6 and members == [0, 1]
    # rank 0 hosts the store: it leaves last
    store.add("bye", 1)
    if rank == 0:
        while int(store.add("bye", 0)) < world:
            time.sleep(0.01)


def test_supervisor_restarts_once_and_resumes(tmp_path):
    script = tmp_path / "job.py"
    script.write_text(textwrap.dedent(f"""
        import json, os, sys, time
        rank, restart = int(os.environ["RANK"]), int(os.environ["MESH_RESTART"])
        ck = "{tmp_path}/ckpt.json"
        start = json.load(open(ck))["step"] if os.path.exists(ck) else 0
        for step in range(start, 6):
            if rank == 1 and restart == 0 and step == 3:
                # the injected failure: a rank exits on the host, once the checkpoint of step 3 is on disk
                t_end = time.time() + 10
                while time.time() < t_end and not (os.path.exists(ck) and json.load(open(ck))["step"] >= 3):
                    time.sleep(0.01)
                sys.exit(7)
            time.sleep(0.05)
            if rank == 0:
                json.dump({{"step": step + 1}}, open(ck + ".tmp", "w")); os.replace(ck + ".tmp", ck)
        open("{tmp_path}/done-%d-%d" % (rank, restart), "w").write(str(start))
    """))
    r = subprocess.run([sys.executable, "-m", "mesh_b200.tools.meshrun", "--nproc", "2", "--max-restarts", "1",
                        "--backoff", "0.2", "--grace", "5", "--", str(script)], cwd=ROOT, capture_output=True, text=True,
                       timeout=120)
    assert r.returncode == 0, r.stderr
    events = [json.loads(l)["event"] for l in r.stderr.splitlines() if l.startswith("{")]
    assert events.count("launched") == 2 and "rank_failed" in events and events[-1] == "finished"
    assert (tmp_path / "done-0-1").exists() and int((tmp_path / "done-1-1").read_text()) >= 3   # resumed, not restarted from 0


def _one_rank_raises(rank, world, rdv):
    if rank == 1:
        raise ValueError("injected failure on rank 1")


def test_a_failed_rank_releases_its_peers_from_the_exit_barrier_at_once():
    """A rank that raises publishes a poison key; the ranks waiting at the end leave with an error in seconds
    rather than after the barrier's full timeout."""
    import time
    from mesh_b200.utils.launch import spawn_ranks
    t0 = time.monotonic()
    with pytest.raises(Exception):
        spawn_ranks(_one_rank_raises, 3, timeout=100.0)
    assert time.monotonic() - t0 < 60.0


_ELASTIC_JOB = '''
import json, os, sys, time
import torch, torch.distributed as dist
sys.path.insert(0, {root!r})
from mesh_b200.ckpt import latest_step, load_sharded, save_sharded
from mesh_b200.compiler.placement import counts

rank, world, restart = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["MESH_RESTART"])
dist.init_process_group("gloo", rank=rank, world_size=world)
ck, ROWS, COLS, STEPS = {ck!r}, 10, 6, 8
g = torch.Generator().manual_seed(0)
X, Y = torch.randn(32, ROWS, generator=g), torch.randn(32, COLS, generator=g)
cnt = counts(ROWS, None, world)
lo = sum(cnt[:rank])
if latest_step(ck) is None:
    W = (torch.randn(ROWS, COLS, generator=g) * 0.1)[lo:lo + cnt[rank]].clone()      # this rank's rows only
    mom, step0 = torch.zeros_like(W), 0
else:
    # the checkpoint was written by another world size: every tensor is re-cut on load
    state, extra = load_sharded(ck, None, rank, world)
    W, mom, step0 = state["W"], state["mom"], extra["step"]
    assert W.shape[0] == cnt[rank]
losses = []
for step in range(step0, STEPS):
    Wf = torch.zeros(ROWS, COLS)
    Wf[lo:lo + cnt[rank]] = W
    try:
        dist.all_reduce(Wf)                  # gathers the row shards (every other rank contributes zeros there)
    except RuntimeError:
        os._exit(75)                         # a peer went away under the collective: not this rank's failure
    Wf.requires_grad_(True)
    loss = (X @ Wf - Y).square().mean()
    loss.backward()
    mom = 0.9 * mom + Wf.grad[lo:lo + cnt[rank]]
    W = W - 0.05 * mom
    losses.append(float(loss))
    save_sharded(ck, step + 1, {{"W": W, "mom": mom}}, {{"W": (0, cnt), "mom": (0, cnt)}}, rank, world,
                 extra={{"step": step + 1}}, barrier=dist.barrier)
    if restart == 0 and rank == world - 1 and step + 1 == 3:
        dist.destroy_process_group()         # leaves between steps, nothing in flight, its checkpoint committed
        sys.exit(9)
if rank == 0:
    json.dump({{"world": world, "first_step": step0, "losses": losses}}, open({out!r}, "w"))
dist.destroy_process_group()
'''


def test_job_is_reformed_at_a_smaller_world_and_resumes_from_its_sharded_checkpoint(tmp_path):
    """Three ranks train with row-sharded weights and momentum; the last rank exits between steps after step 3; the
    supervisor re-forms the job with two ranks, which load the three-way checkpoint re-cut two ways and continue at
    step 3: their losses equal those of an uninterrupted run."""
    import torch
    script = tmp_path / "job.py"
    script.write_text(_ELASTIC_JOB.format(root=ROOT, ck=str(tmp_path / "ck"), out=str(tmp_path / "out.json")))
    r = subprocess.run([sys.executable, "-m", "mesh_b200.tools.meshrun", "--nproc", "3", "--max-restarts", "1", "--shrink",
                        "--backoff", "0.2", "--grace", "10", "--", str(script)], cwd=ROOT, capture_output=True, text=True,
                       timeout=240)
    assert r.returncode == 0, r.stderr[-3000:]
    events = [json.loads(l) for l in r.stderr.splitlines() if l.startswith("{")]
    launched = [e["nproc"] for e in events if e["event"] == "launched"]
    assert launched == [3, 2] and events[-1]["event"] == "finished"
    out = json.load(open(tmp_path / "out.json"))
    assert out["world"] == 2 and out["first_step"] == 3 and len(out["losses"]) == 5
    # the uninterrupted run, in one process
    g = torch.Generator().manual_seed(0)
    X, Y = torch.randn(32, 10, generator=g), torch.randn(32, 6, generator=g)
    W = torch.randn(10, 6, generator=g) * 0.1
    mom, want = torch.zeros_like(W), []
    for _ in range(8):
        Wf = W.clone().requires_grad_(True)
        loss = (X @ Wf - Y).square().mean()
        loss.backward()
        mom = 0.9 * mom + Wf.grad
        W = W - 0.05 * mom
        want.append(float(loss))
    assert out["losses"] == pytest.approx(want[3:], rel=1e-5)
