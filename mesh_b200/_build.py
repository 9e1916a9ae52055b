"""In-tree build of the native library (``mesh_b200/_lib/libmesh_b200.so``).

Every ``.cu`` / ``.cpp`` under ``mesh_b200/csrc`` is compiled with nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and linked into one shared object that
Python loads through ctypes.  Objects are cached by content hash, so a rebuild after a
small edit takes seconds.  Run ``python -m mesh_b200._build`` or call :func:`build`.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import json
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "_lib"
OBJDIR = ROOT.parent / "build" / "obj"
LIBNAME = "libmesh_b200.so"
CHECK_LIBNAME = "libmesh_b200_check.so"      # same sources with -DMESH_CHECK=1 (index / alignment checks in the kernels)

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=default", "--expt-relaxed-constexpr", "-DNDEBUG",
]


def nvcc_path() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def sources() -> list[Path]:
    out = sorted(p for p in CSRC.rglob("*.cu")) + sorted(p for p in CSRC.rglob("*.cpp"))
    return [p for p in out if "/standalone/" not in str(p)]


def _flags(check: bool) -> list[str]:
    return NVCC_FLAGS + (["-DMESH_CHECK=1"] if check else [])


def _headers_digest(check: bool = False) -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))):
        h.update(p.read_bytes())
    h.update(" ".join(_flags(check)).encode())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, hdr: str, verbose: bool, check: bool = False) -> Path:
    h = hashlib.sha256(src.read_bytes())
    h.update(hdr.encode())
    obj = OBJDIR / f"{src.stem}-{h.hexdigest()[:16]}.o"
    if obj.exists():
        return obj
    cmd = [nvcc, *_flags(check), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cpp":
        cmd.insert(1, "-x"); cmd.insert(2, "cu")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        print(r.stderr, file=sys.stderr)
    return obj


def lib_path(check: bool = False) -> Path:
    return LIBDIR / (CHECK_LIBNAME if check else LIBNAME)


def _meta_path(check: bool) -> Path:
    return LIBDIR / ("build_check.json" if check else "build.json")


def is_current(check: bool = False) -> bool:
    meta = _meta_path(check)
    if not (lib_path(check).exists() and meta.exists()):
        return False
    try:
        return json.loads(meta.read_text()).get("digest") == _tree_digest(check)
    except Exception:
        return False


def _tree_digest(check: bool = False) -> str:
    h = hashlib.sha256(_headers_digest(check).encode())
    for s in sources():
        h.update(str(s.relative_to(CSRC)).encode())
        h.update(s.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, check: bool = False) -> Path:
    """Compile every source for sm_100a and link the shared library.  Returns its path.
    ``check=True`` builds the checked variant (``-DMESH_CHECK=1``) beside the regular one."""
    if not force and is_current(check):
        return lib_path(check)
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build mesh_b200's native library")
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    # one builder at a time: the ranks of a job that all find the library stale take turns, and all but the first
    # find it current when their turn comes
    import fcntl
    with open(LIBDIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and is_current(check):
            return lib_path(check)
        return _build_locked(nvcc, verbose, check)


def _build_locked(nvcc: str, verbose: bool, check: bool) -> Path:
    hdr = _headers_digest(check)
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(lambda s: _compile_one(nvcc, s, hdr, verbose, check), srcs))
    tmp = LIBDIR / (lib_path(check).name + ".tmp")
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(tmp),
           *map(str, objs), "-lpthread", "-ldl", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib_path(check))
    _meta_path(check).write_text(json.dumps({"digest": _tree_digest(check), "sources": [str(s.relative_to(CSRC)) for s in srcs],
                                             "objects": [o.name for o in objs]}))
    _prune_objects()
    return lib_path(check)


def _prune_objects() -> None:
    """Objects are cached by content hash; those that neither library variant was last linked from are deleted, so the
    cache does not grow with every edit."""
    keep: set[str] = set()
    for check in (False, True):
        try:
            keep.update(json.loads(_meta_path(check).read_text()).get("objects", []))
        except Exception:
            return                                  # an older metadata file: keep everything
    for f in OBJDIR.glob("*.o"):
        if f.name not in keep:
            try:
                f.unlink()
            except OSError:
                pass


RACE_CHECK_SOURCES = ["runtime/runtime.cpp", "runtime/host_engine.cpp", "standalone/race_check.cpp"]


def build_race_check(out: Path | None = None) -> Path | None:
    """The host runtime's thread-facing sources and their driver (``csrc/standalone/race_check.cpp``) compiled with
    ThreadSanitizer into one executable.  ``None`` when the compiler has no ThreadSanitizer runtime."""
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        return None
    out = out or (ROOT.parent / "build" / "race_check")
    out.parent.mkdir(parents=True, exist_ok=True)
    cmd = [cxx, "-std=c++17", "-fsanitize=thread", "-O1", "-g", "-pthread", *[str(CSRC / f) for f in RACE_CHECK_SOURCES],
           "-o", str(out), "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        if "tsan" in r.stderr.lower() or "sanitize" in r.stderr.lower():
            return None
        raise RuntimeError(f"race check did not compile:\n{r.stderr[-2000:]}")
    return out


def run_race_check(timeout: float = 300.0) -> tuple[int, str]:
    """Build and run the race check: ``(exit code, output)``; 0 = the driver's expectations held and ThreadSanitizer
    reported nothing, 66 = ThreadSanitizer reported a race, -1 = no ThreadSanitizer here."""
    exe = build_race_check()
    if exe is None:
        return -1, "no ThreadSanitizer runtime"
    env = dict(os.environ, TSAN_OPTIONS="exitcode=66 halt_on_error=0")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=timeout, env=env)
    return r.returncode, (r.stdout + r.stderr)[-6000:]


if __name__ == "__main__":
    if "--race-check" in sys.argv:
        rc, text = run_race_check()
        print(text)
        sys.exit(0 if rc in (0, -1) else rc)
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv, check="--check" in sys.argv)
    print(p)
