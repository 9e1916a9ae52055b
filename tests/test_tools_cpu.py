"""Ops tools on CPU with fakes: telemetry provider, preflight probe, peer discovery, runtime identity, hourly runner."""
import json
import sys
import types
import urllib.request

from mesh_b200.tools import hourly, peers, preflight, runtime_id, telemetry


class FakeGpuSource:
    def __init__(self):
        self.n = 0

    def sample(self):
        self.n += 1
        return [{"gpu": 0, "sm_mhz": 1900 + self.n, "power_w": 400.0, "util_pct": 90, "mem_used_mb": 1000, "throttle": 0}]


def test_telemetry_ring_leases_and_http():
    p = telemetry.Provider(FakeGpuSource(), interval_s=0.01, ring=4)
    for _ in range(6):
        p.tick()
    code, body = p.handle("GET", "/samples?since=0")
    assert code == 200 and len(body["samples"]) == 4 and body["missed"] == 2 and body["next"] == 6
    code, body = p.handle("GET", f"/samples?since={body['next']}")
    assert body["samples"] == [] and body["missed"] == 0
    code, body = p.handle("POST", "/workload", json.dumps({"name": "ffn", "flops": 1e12, "seconds": 1e-3}).encode())
    assert code == 200
    assert p.handle("GET", "/workloads")[1]["workloads"][0]["name"] == "ffn"
    assert p.handle("GET", "/nope")[0] == 404
    srv = telemetry.serve(p, "127.0.0.1", 0)
    import threading
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    url = f"http://127.0.0.1:{srv.server_address[1]}"
    assert json.loads(urllib.request.urlopen(url + "/health", timeout=5).read())["ok"]
    got = json.loads(urllib.request.urlopen(url + "/samples?since=4", timeout=5).read())
    assert [s["gpus"][0]["sm_mhz"] for s in got["samples"]] == [1905, 1906]
    srv.shutdown()


def _fake_nvml(free_mib, procs):
    m = types.SimpleNamespace()
    m.nvmlDeviceGetCount = lambda: len(free_mib)
    m.nvmlDeviceGetHandleByIndex = lambda i: i
    m.nvmlDeviceGetMemoryInfo = lambda h: types.SimpleNamespace(free=free_mib[h] << 20, total=183359 << 20)
    m.nvmlDeviceGetComputeRunningProcesses = lambda h: [types.SimpleNamespace(pid=p, usedGpuMemory=512 << 20) for p in procs.get(h, [])]
    m.nvmlDeviceGetName = lambda h: b"NVIDIA B200"
    return m


def test_preflight_reports_collisions():
    full = [[True] * 2 for _ in range(2)]
    absent = [{"rank": r, "state": "absent"} for r in range(2)]
    ok = preflight.probe(2, nvml=_fake_nvml([180000, 180000], {}), peers=full, blocks=absent)
    assert ok["ok"] and ok["problems"] == []
    bad = preflight.probe(2, nvml=_fake_nvml([180000, 4000], {0: [4242]}), peers=[[True, False], [True, True]],
                          blocks=[{"rank": 0, "state": "live", "pid": 7}, {"rank": 1, "state": "stale", "pid": 8}], min_free_mib=8192)
    text = " | ".join(bad["problems"])
    assert not bad["ok"] and "pid 4242" in text and "4000 MiB free" in text and "0-1" in text and "in use" in text
    assert bad["stale_ranks"] == [1]
    assert "3 ranks wanted" in " ".join(preflight.probe(3, nvml=_fake_nvml([180000] * 2, {}), peers=full, blocks=absent)["problems"])


def test_peer_discovery_topology_and_islands():
    # GPUs 0-3 and 4-5 form two islands
    acc = lambda a, b: (a < 4) == (b < 4)
    f = peers.discover(6, acc, {"nvlink_p2p_gbs": 770.0})
    assert not f["all_connected"] and peers.islands(f) == [[0, 1, 2, 3], [4, 5]]
    topo = peers.topology(f)
    assert len(topo.between(0, 3)) == 1 and topo.between(3, 4) == []
    assert abs(topo.between(0, 1)[0].bandwidth - 770e9 * 8 / 5) < 1


def test_runtime_identity_matches_itself():
    a, b = runtime_id.identity(), runtime_id.identity()
    assert a["native_library"]["present"] and runtime_id.same([a, b]) == []
    c = dict(b, torch="0.0")
    assert runtime_id.same([a, c]) == ["torch"]


def test_hourly_runner_records_result_failure_and_timeout(tmp_path):
    py = sys.executable
    ok = hourly.run_one({"name": "ok", "cmd": [py, "-c", "print('x'); print('{\"value\": 3}')"], "deadline_s": 30}, cwd=tmp_path)
    assert ok["status"] == "ok" and ok["result"] == {"value": 3}
    bad = hourly.run_one({"name": "bad", "cmd": [py, "-c", "import sys; print('boom'); sys.exit(3)"], "deadline_s": 30}, cwd=tmp_path)
    assert bad["status"] == "exit 3" and "boom" in bad["tail"]
    slow = hourly.run_one({"name": "slow", "cmd": [py, "-c", "import time; time.sleep(60)"], "deadline_s": 1}, cwd=tmp_path)
    assert slow["status"] == "timeout" and slow["seconds"] < 20


def test_micro_workloads_run_small_and_variants_agree():
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "micro.py")
    spec = importlib.util.spec_from_file_location("micro_workloads", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    recs = mod.main(["all", "--small", "--device", "cpu", "--steps", "1"])
    names = {r["workload"] for r in recs}
    assert names == set(mod.WORKLOADS)
    assert all(r["ms"] > 0 for r in recs)
    assert all(r["orthogonality_error"] < 1e-3 for r in recs if r["workload"] == "orth")
    assert all(r.get("difference", 0) < 1e-4 for r in recs if r["workload"] in ("pairwise", "moe_dispatch"))
