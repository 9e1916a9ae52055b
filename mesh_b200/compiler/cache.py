"""Cache of compiled programs on disk, so that a job that starts again does not export and place its model again.

The key covers everything the result depends on: the module's structure and the shapes and dtypes of its state, the
example arguments' shapes and dtypes, the processors and grid, the compile options, what the placement callable says
about every parameter and input name, and the sources of this compiler.  A hit loads the archive
(``archive.load``); a miss compiles and saves.  The reference keeps compiled programs as "serialized objects we can
resume without re-compiling" (rdma/mesh_compile.py:8398-8400; compiler/mesh_compiler/archive.py:24-83); this adds the
key and the lookup.
"""
from __future__ import annotations

import hashlib
import inspect
import json
import os
from pathlib import Path

import torch

from . import archive
from .driver import compile_module


class _Probe:
    """Stands in for a graph placeholder when asking a placement what it would say about a name."""

    def __init__(self, name, value):
        self.op, self.name, self.target = "placeholder", name, name
        self.meta = {"val": value}
        self.args, self.kwargs = (), {}


def _placement_signature(placement, module: torch.nn.Module, arg_names: list[str], args) -> list:
    out = []
    names = [("p_" + n.replace(".", "_"), p) for n, p in module.named_parameters()]
    names += [("b_" + n.replace(".", "_"), b) for n, b in module.named_buffers()]
    names += list(zip(arg_names, args))
    for name, value in names:
        try:
            said = placement(_Probe(name, value if isinstance(value, torch.Tensor) else None))
        except Exception as e:            # a placement that needs a real graph node: fall back to its source text
            said = f"<{type(e).__name__}>"
        out.append((name, repr(said)))
    try:
        out.append(("source", inspect.getsource(placement)))
    except (OSError, TypeError):
        out.append(("source", getattr(placement, "__qualname__", repr(type(placement)))))
    return out


def _compiler_version() -> str:
    h = hashlib.sha256()
    for p in sorted(Path(__file__).parent.glob("*.py")):
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def cache_key(module, args, processors, placement, mesh=None, **options) -> str:
    try:
        arg_names = [n for n in inspect.signature(module.forward).parameters][: len(args)]
    except (TypeError, ValueError):
        arg_names = [f"arg{i}" for i in range(len(args))]
    desc = {
        "module": repr(module),
        "state": [(n, tuple(t.shape), str(t.dtype)) for n, t in list(module.named_parameters()) + list(module.named_buffers())],
        "args": [(tuple(a.shape), str(a.dtype)) if isinstance(a, torch.Tensor) else repr(a) for a in args],
        "processors": [(k, tuple(v)) for k, v in processors.items()],
        "mesh": tuple(mesh) if mesh else None,
        "options": sorted((k, repr(v)) for k, v in options.items()),
        "placement": _placement_signature(placement, module, arg_names, args),
        "compiler": _compiler_version(),
        "torch": torch.__version__,
    }
    return hashlib.sha256(json.dumps(desc, sort_keys=True, default=str).encode()).hexdigest()[:24]


def compile_cached(module, args, processors, placement, cache_dir: str | os.PathLike, mesh=None, **options):
    """``compile_module`` through the cache.  Returns ``(scheduled, hit)``."""
    key = cache_key(module, args, processors, placement, mesh, **options)
    where = Path(cache_dir) / key
    if (where / "scheduled.json").exists() or (where / "state.pt").exists() or (where.exists() and any(where.iterdir())):
        try:
            return archive.load(str(where)), True
        except Exception:
            pass                              # an unreadable entry is compiled again and overwritten
    sch = compile_module(module, args, processors, placement, mesh=mesh, **options)
    from ..utils.disk import room
    room(str(cache_dir), 1 << 20)
    where.mkdir(parents=True, exist_ok=True)
    archive.save(str(where), sch)
    return sch, False
