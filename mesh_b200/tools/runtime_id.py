"""Identity of the software a rank runs: ``python -m mesh_b200.tools.runtime_id`` prints one JSON object.

Ranks of one job must run the same interpreter, torch, CUDA runtime and native library; comparing this record across
ranks (or nodes) before a run finds the mismatch that would otherwise show up as a hang or a wrong plan signature
(the reference reports its runtime's lock-file hash, interpreter and packages the same way, bin/mesh-runtime-id.py)."""
from __future__ import annotations

import hashlib
import json
import platform
import sys
from pathlib import Path


def identity() -> dict:
    import torch
    root = Path(__file__).resolve().parents[1]
    h = hashlib.sha256()
    for p in sorted((root / "csrc").rglob("*")):
        if p.suffix in (".cu", ".cuh", ".cpp", ".h"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    lib = root / "_lib" / "libmesh_b200.so"
    py = hashlib.sha256()
    for p in sorted(root.rglob("*.py")):
        py.update(p.read_bytes())
    return {"python": sys.version.split()[0], "platform": platform.platform(), "torch": torch.__version__,
            "cuda": torch.version.cuda, "nccl": ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None,
            "native_sources_sha256": h.hexdigest()[:16], "python_sources_sha256": py.hexdigest()[:16],
            "native_library": {"present": lib.exists(), "bytes": lib.stat().st_size if lib.exists() else 0}}


def same(records: list[dict], keys=("python", "torch", "cuda", "native_sources_sha256", "python_sources_sha256")) -> list[str]:
    """Keys on which the records differ (empty: the ranks match)."""
    return [k for k in keys if len({json.dumps(r.get(k)) for r in records}) > 1]


if __name__ == "__main__":
    print(json.dumps(identity()))
