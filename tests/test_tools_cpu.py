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


def test_observer_merges_providers_and_reports_a_silent_node():
    import json
    import threading
    import urllib.request
    from mesh_b200.tools import observe, telemetry

    class Fake:
        def __init__(self, n):
            self.n = n

        def sample(self):
            return [{"gpu": i, "util_pct": 50, "power_w": 400.0, "mem_used_mb": 1000} for i in range(self.n)]

    servers, nodes = [], {}
    for name, n in (("a", 2), ("b", 4)):
        p = telemetry.Provider(Fake(n))
        p.tick()
        p.handle("POST", "/workload", json.dumps({"name": "ffn", "seconds": 0.5, "flops": 1e12, "hbm_bytes": 1e9}).encode())
        srv = telemetry.serve(p, "127.0.0.1", 0)
        threading.Thread(target=srv.serve_forever, daemon=True).start()
        servers.append(srv)
        nodes[name] = f"http://127.0.0.1:{srv.server_address[1]}"
    nodes["gone"] = "http://127.0.0.1:9"                                   # nothing listens there
    ob = observe.Observer(nodes, timeout_s=0.5)
    ob.poll()
    m = ob.merged()
    assert m["nodes"]["a"]["fresh"] and m["nodes"]["b"]["gpus"] == 4 and m["nodes"]["a"]["mean_util"] == 50
    assert not m["nodes"]["gone"]["ok"] and m["nodes"]["gone"]["error"]
    t = m["totals"]
    assert t["nodes"] == 3 and t["nodes_ok"] == 2 and t["gpus"] == 6 and abs(t["power_w"] - 2400.0) < 1e-6
    assert abs(t["flops_per_s"] - 4e12) < 1 and abs(t["bytes_per_s"] - 4e9) < 1
    ob.poll()                                                             # cursors advanced: no workload is counted twice
    assert ob.merged()["nodes"]["a"]["workloads"] == 0
    web = observe.serve(ob, "127.0.0.1", 0)
    threading.Thread(target=web.serve_forever, daemon=True).start()
    base = f"http://127.0.0.1:{web.server_address[1]}"
    assert json.loads(urllib.request.urlopen(base + "/mesh.json", timeout=2).read())["totals"]["gpus"] == 6
    assert b"<table" in urllib.request.urlopen(base + "/", timeout=2).read()
    for s in servers + [web]:
        s.shutdown()


def test_application_bundle_pack_verify_unpack_push(tmp_path):
    import io
    import shutil
    import tarfile
    from mesh_b200.tools import application as app
    src = tmp_path / "app"
    (src / "pkg" / "__pycache__").mkdir(parents=True)
    (src / "pkg" / "main.py").write_text("print('hello')\n")
    (src / "pkg" / "__pycache__" / "junk.pyc").write_bytes(b"x")
    (src / "data.bin").write_bytes(bytes(range(256)) * 64)
    man = app.pack(src, tmp_path / "app.tar.gz")
    assert set(man["files"]) == {"pkg/main.py", "data.bin"} and man["total_bytes"] == 15 + 256 * 64
    assert app.manifest(src)["digest"] == man["digest"] == app.read_manifest(tmp_path / "app.tar.gz")["digest"]
    assert app.verify(tmp_path / "app.tar.gz") == []
    app.unpack(tmp_path / "app.tar.gz", tmp_path / "out")
    assert (tmp_path / "out" / "pkg" / "main.py").read_text() == "print('hello')\n" and app.verify(tmp_path / "out") == []
    (tmp_path / "out" / "data.bin").write_bytes(b"changed")
    (tmp_path / "out" / "new.txt").write_text("x")
    assert sorted(app.verify(tmp_path / "out")) == ["changed: data.bin", "extra: new.txt"]
    (src / "pkg" / "main.py").write_text("print('other')\n")
    assert app.manifest(src)["digest"] != man["digest"]                      # other bytes, other digest
    # a member that would leave the destination is refused
    bad = tmp_path / "bad.tar.gz"
    with tarfile.open(bad, "w:gz") as tar:
        data = b'{"files": {}, "digest": "", "total_bytes": 0}'
        info = tarfile.TarInfo(app.MANIFEST)
        info.size = len(data)
        tar.addfile(info, io.BytesIO(data))
        info = tarfile.TarInfo("../escape.txt")
        info.size = 1
        tar.addfile(info, io.BytesIO(b"x"))
    import pytest
    with pytest.raises(Exception):
        app.unpack(bad, tmp_path / "jail")
    assert not (tmp_path / "escape.txt").exists()

    def local(host, bundle, dest):
        if host == "down":
            raise ConnectionError("no route")
        app.unpack(bundle, tmp_path / host / dest.lstrip("/"))
    rep = app.push(tmp_path / "app.tar.gz", "/opt/app", ["n1", "down", "n2"], transport=local)
    assert rep["digest"] == man["digest"] and rep["hosts"]["n1"] == rep["hosts"]["n2"] == "ok" and "no route" in rep["hosts"]["down"]
    assert app.verify(tmp_path / "n2" / "opt" / "app") == []
    shutil.rmtree(tmp_path / "n1")


def test_fleet_run_selects_nodes_bounds_each_and_reports(tmp_path):
    import subprocess
    import sys
    from mesh_b200.tools import fleet
    hosts_file = tmp_path / "nodes.txt"
    hosts_file.write_text("# the job's nodes\nn1 10.0.0.1\nn2\nslow 10.0.0.3  # takes too long\n")
    hosts = fleet.read_hosts(hosts_file)
    assert hosts == {"n1": "10.0.0.1", "n2": "n2", "slow": "10.0.0.3"}
    assert set(fleet.select(hosts, "others", me="n2")) == {"n1", "slow"} and list(fleet.select(hosts, "n1,slow")) == ["n1", "slow"]
    import pytest
    with pytest.raises(KeyError):
        fleet.select(hosts, "nope")

    def runner(address, command, deadline):
        if address == "10.0.0.3":
            raise subprocess.TimeoutExpired(command, deadline)
        if address == "n2":
            return 3, "", "boom"
        return 0, f"{address}: {' '.join(command)}", ""
    seen = []
    res = fleet.run(hosts, ["echo", "hi"], deadline_s=0.5, runner=runner, emit=lambda n, r: seen.append(n))
    assert res["n1"]["status"] == "ok" and res["n1"]["stdout"] == "10.0.0.1: echo hi"
    assert res["n2"]["status"] == "failed" and res["n2"]["code"] == 3 and res["slow"]["status"] == "timeout"
    assert sorted(seen) == ["n1", "n2", "slow"]
    # a real local command through the default runner
    out = fleet.run({"here": "localhost"}, [sys.executable, "-c", "print(6 * 7)"], deadline_s=30)
    assert out["here"]["status"] == "ok" and out["here"]["stdout"].strip() == "42"

    def identities(address, command, deadline):
        import json
        rec = {"python": "3.12", "torch": "2.11", "cuda": "12.8", "native_sources_sha256": "a" if address == "n2" else "b",
               "python_sources_sha256": "c"}
        return 0, json.dumps(rec), ""
    rep = fleet.status({"n1": "n1", "n2": "n2"}, runner=identities)
    assert rep["differ_on"] == ["native_sources_sha256"] and not rep["unreachable"]
