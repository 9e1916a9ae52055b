"""One configuration object for the whole runtime (env ``MESH_*`` + keyword overrides).

Mirrors the reference's scattered configuration surface — ``MESH_GROUP`` / ``MESH_PROGRAM`` /
``MESH_LEDGER`` / ``MESH_DEADLINE`` environment variables (rdma/mesh_compile.py:1810-1832),
``etc/bridge.conf`` key=value pairs and the compile-time ``MESH_PLATFORM_NS`` wait bound
(rdma/Makefile:6-7) — in a single dataclass.
"""
from __future__ import annotations

import dataclasses
import json
import os
from pathlib import Path
from typing import Any


def _env(name: str, default: Any, cast=str):
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    if cast is bool:
        return v.lower() in ("1", "true", "yes", "on")
    return cast(v)


@dataclasses.dataclass
class MeshConfig:
    group: str = "mesh"                 # run id, identical on every rank (MESH_GROUP)
    program: str = ""                   # comma list of rank indices that take part (MESH_PROGRAM)
    ledger: bool = False                # per-signal/wait device timestamps (MESH_LEDGER)
    check: bool = False                 # bounds/alignment-checked kernels (MESH_CHECK)
    wait_ns: int = 5_000_000_000        # host-side "no progress" bound, like MESH_PLATFORM_NS (5 s)
    device_wait_ns: int = 2_000_000_000 # device-side bounded waits
    deadline_s: float = 0.0             # whole-run deadline, 0 = none (MESH_DEADLINE)
    heap_bytes: int = 4 << 30           # symmetric heap size per GPU (MESH_HEAP_BYTES)
    signal_bytes: int = 1 << 20         # signal pad size per GPU
    one_shot_max_bytes: int = 512 << 10 # all-reduce: one-shot below, two-shot above
    nvls: bool = True                   # use NVLS multimem paths when the heap has a multicast mapping
    metrics_path: str = ""              # JSON-lines step log (MESH_METRICS)
    capacity_path: str = ""             # roofline operands (defaults to MEASURED_PEAKS.json / built-in)
    heartbeat_s: float = 1.0
    restart_backoff_s: float = 60.0     # the supervisor reopens at most once per interval

    @classmethod
    def from_env(cls, **overrides) -> "MeshConfig":
        c = cls(
            group=_env("MESH_GROUP", cls.group),
            program=_env("MESH_PROGRAM", cls.program),
            ledger=_env("MESH_LEDGER", cls.ledger, bool),
            check=_env("MESH_CHECK", cls.check, bool),
            wait_ns=_env("MESH_WAIT_NS", cls.wait_ns, int),
            device_wait_ns=_env("MESH_DEVICE_WAIT_NS", cls.device_wait_ns, int),
            deadline_s=_env("MESH_DEADLINE", cls.deadline_s, float),
            heap_bytes=_env("MESH_HEAP_BYTES", cls.heap_bytes, int),
            signal_bytes=_env("MESH_SIGNAL_BYTES", cls.signal_bytes, int),
            one_shot_max_bytes=_env("MESH_ONE_SHOT_MAX", cls.one_shot_max_bytes, int),
            nvls=_env("MESH_NVLS", cls.nvls, bool),
            metrics_path=_env("MESH_METRICS", cls.metrics_path),
            capacity_path=_env("MESH_CAPACITY", cls.capacity_path),
            heartbeat_s=_env("MESH_HEARTBEAT_S", cls.heartbeat_s, float),
            restart_backoff_s=_env("MESH_RESTART_BACKOFF_S", cls.restart_backoff_s, float),
        )
        return dataclasses.replace(c, **overrides)

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), sort_keys=True)


_config: MeshConfig | None = None


def config() -> MeshConfig:
    """Process-wide configuration, read from the environment on first use."""
    global _config
    if _config is None:
        _config = MeshConfig.from_env()
    return _config


def set_config(c: MeshConfig) -> None:
    global _config
    _config = c


# Measured peaks of one B200 in this deployment; overridden by a MEASURED_PEAKS.json next to the
# package or by MESH_CAPACITY.  Plays the role of the reference's etc/mesh-capacity.json.
DEFAULT_CAPACITY = {
    "hbm_gbs": 6529.7,
    "bf16_tflops": 1648.0,
    "bf16_tflops_sustained": 1382.0,
    "nvlink_gbs_per_dir": 770.0,
    "nvlink_allreduce_busbw_gbs": 725.0,
    "sm_count": 148,
}


def capacity() -> dict:
    cap = dict(DEFAULT_CAPACITY)
    paths = []
    if config().capacity_path:
        paths.append(Path(config().capacity_path))
    paths.append(Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json")
    for p in paths:
        try:
            cap.update({k: v for k, v in json.loads(p.read_text()).items() if isinstance(v, (int, float))})
            break
        except Exception:
            continue
    return cap
