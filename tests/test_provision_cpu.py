"""Node convergence (``mesh_b200/tools/provision.py``): reports, applies under a staging root, is idempotent, and never
calls a setter of a GPU's settings."""
import json
import types


class _FakeNvml(types.SimpleNamespace):
    """A pynvml-like module that records every call; any ``nvmlDeviceSet*`` call is a test failure."""

    def __init__(self, n):
        super().__init__()
        self.n, self.calls = n, []

    def __getattr__(self, name):
        if name.startswith("nvmlDeviceSet") or name.startswith("nvmlDeviceReset"):
            raise AssertionError(f"provisioning tried to change a GPU setting: {name}")
        raise AttributeError(name)

    def nvmlDeviceGetCount(self):
        return self.n

    def nvmlDeviceGetHandleByIndex(self, i):
        return i

    def nvmlDeviceGetMemoryInfo(self, h):
        return types.SimpleNamespace(free=170 << 30, total=180 << 30)

    def nvmlDeviceGetComputeRunningProcesses(self, h):
        return []

    def nvmlDeviceGetName(self, h):
        return "NVIDIA B200"

    def nvmlDeviceGetPersistenceMode(self, h):
        self.calls.append("persistence")
        return 1

    def nvmlDeviceGetPowerManagementLimit(self, h):
        self.calls.append("power")
        return 1000000


def test_provision_reports_then_converges_and_is_idempotent(tmp_path):
    from mesh_b200.tools import provision as P
    keys = tmp_path / "fleet.pub"
    keys.write_text("ssh-ed25519 AAAA fleet@a")
    root = tmp_path / "root"
    items = P.desired(2, str(keys))
    assert {i.path for i in items} >= {"/etc/mesh_b200/env", "/etc/systemd/system/mesh-telemetry.service",
                                       "/etc/systemd/system/mesh-hourly.timer", "/etc/ssh/authorized_keys.d/mesh_fleet"}
    first = P.diff(items, root)
    assert len(first) == len(items) and all(c["change"] == "create" for c in first)
    assert not root.exists()                                   # a report writes nothing
    done = P.apply(items, root)
    assert len(done) == len(items)
    assert (root / "etc/ssh/authorized_keys.d/mesh_fleet").stat().st_mode & 0o777 == 0o600
    assert "mesh_b200.tools.telemetry" in (root / "etc/systemd/system/mesh-telemetry.service").read_text()
    assert P.diff(items, root) == [] and P.apply(items, root) == []          # converged: nothing left to do
    (root / "etc/mesh_b200/env").write_text("MESH_GPUS=1\n")                   # drift is found and repaired
    assert [c["change"] for c in P.diff(items, root)] == ["rewrite"]
    P.apply(items, root)
    assert P.diff(items, root) == []


def test_provision_only_reads_gpu_settings():
    from mesh_b200.tools import provision as P
    nvml = _FakeNvml(2)
    facts = P.checks(2, nvml)
    by = {f["check"]: f for f in facts}
    assert by["2 GPU(s) visible"]["ok"] and by["2 GPU(s) visible"]["seen"] == 2
    assert by["GPU settings (read only, never changed)"]["seen"] == [
        {"gpu": 0, "persistence": 1, "power_limit_mw": 1000000}, {"gpu": 1, "persistence": 1, "power_limit_mw": 1000000}]
    assert set(nvml.calls) == {"persistence", "power"}
    assert not P.checks(4, nvml)[-2]["ok"]                      # asks for more GPUs than there are


def test_provision_cli_exit_codes(tmp_path, capsys, monkeypatch):
    from mesh_b200.tools import provision as P
    monkeypatch.setattr(P, "checks", lambda gpus, nvml=None: [{"check": "stub", "ok": True, "seen": None}])
    assert P.main(["--root", str(tmp_path / "r"), "--gpus", "1"]) == 1            # differs, nothing written
    assert P.main(["--root", str(tmp_path / "r"), "--gpus", "1", "--apply"]) == 0
    assert P.main(["--root", str(tmp_path / "r"), "--gpus", "1"]) == 0            # converged
    out = capsys.readouterr().out
    assert json.loads(out[out.rindex('{\n "root"'):])["changes"] == []
