"""Every name of this package that a test, a benchmark, an example, a model or a driver hook imports must exist.

The GPU tests and the models import names that no CPU test touches; a name deleted from the package would otherwise
only fail on a GPU box.  This test parses every such file with ``ast`` and resolves each ``from mesh_b200... import
name`` (at module level or inside a function) against the package as imported on a CPU-only machine.
"""
import ast
import importlib
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _files():
    out = [ROOT / "__graft_entry__.py", ROOT / "bench.py"]
    for d in ("tests", "benchmarks", "examples", "baseline", "mesh_b200"):
        out += [p for p in sorted((ROOT / d).rglob("*.py")) if "_ref" not in p.parts and "__pycache__" not in p.parts]
    return [p for p in out if p.exists()]


def _package_of(path: Path) -> str:
    rel = path.relative_to(ROOT).with_suffix("")
    parts = list(rel.parts)
    if parts[-1] == "__init__":
        return ".".join(parts[:-1])
    return ".".join(parts[:-1])


def _imports(path: Path):
    tree = ast.parse(path.read_text(), filename=str(path))
    for node in ast.walk(tree):
        if isinstance(node, ast.ImportFrom):
            mod = node.module or ""
            if node.level:
                base = _package_of(path).split(".")
                if path.name == "__init__.py":
                    base = base + []
                base = base[:len(base) - (node.level - 1)] if node.level > 1 else base
                mod = ".".join([*base, mod] if mod else base)
            if mod == "mesh_b200" or mod.startswith("mesh_b200."):
                for alias in node.names:
                    yield mod, alias.name, node.lineno
        elif isinstance(node, ast.Import):
            for alias in node.names:
                if alias.name == "mesh_b200" or alias.name.startswith("mesh_b200."):
                    yield alias.name, None, node.lineno


def _wanted():
    seen = {}
    for path in _files():
        for mod, name, line in _imports(path):
            seen.setdefault((mod, name), f"{path.relative_to(ROOT)}:{line}")
    return sorted(seen.items(), key=lambda kv: (kv[0][0], kv[0][1] or ""))


@pytest.mark.parametrize("key,where", _wanted(), ids=lambda v: f"{v[0]}.{v[1]}" if isinstance(v, tuple) else None)
def test_imported_name_exists(key, where):
    mod, name = key
    module = importlib.import_module(mod)
    if name is None or name == "*":
        return
    if hasattr(module, name):
        return
    try:
        importlib.import_module(f"{mod}.{name}")          # ``from package import submodule``
    except ImportError:
        pytest.fail(f"{where} imports {name!r} from {mod}, which does not define it")


def test_nvtx_ranges_are_balanced_and_off_by_default(monkeypatch):
    """``MESH_NVTX=1`` brackets launches with NVTX ranges; off, nothing touches the NVTX calls."""
    import torch

    from mesh_b200 import _native
    calls = []
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: calls.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: calls.append(("pop", None)))
    monkeypatch.setattr(_native.nvtx, "enabled", False)
    with _native.nvtx("quiet"):
        pass
    assert calls == []
    monkeypatch.setattr(_native.nvtx, "enabled", True)
    with _native.nvtx("outer"):
        with _native.nvtx("inner"):
            pass
    assert calls == [("push", "outer"), ("push", "inner"), ("pop", None), ("pop", None)]
