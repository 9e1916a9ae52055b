"""ctypes access to ``libmesh_b200.so``.

The library is built in-tree by :mod:`mesh_b200._build`.  On a machine with a GPU a missing
or unloadable library is an error (ops never fall back silently to eager PyTorch); on a
machine without one, CPU-only parts of the package work without it.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_int, c_longlong, c_uint32, c_void_p

_lock = threading.Lock()
_lib = None
launch_count = 0   # kernels of this library launched by this process (bench accounting)


on_launch = None   # set by the runtime service: mirrors the count into the process's stats block


def count_launch(n: int = 1) -> None:
    global launch_count
    launch_count += n
    if on_launch is not None:
        on_launch(n)


class nvtx:
    """``with nvtx("name"):`` opens an NVTX range around the block when ``MESH_NVTX=1`` (ranges show up in any tool
    that reads NVTX; off, the block costs one environment lookup at import).  The reference brackets its phases for its
    own ledger (``MESH_LEDGER``); these are the same phases named for external profilers."""
    enabled = __import__("os").environ.get("MESH_NVTX", "0") == "1"

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if nvtx.enabled:
            import torch
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if nvtx.enabled:
            import torch
            torch.cuda.nvtx.range_pop()
        return False


MAX_RANKS = 8


class GemmArgs(ctypes.Structure):
    """Mirror of ``MeshGemmArgs`` (csrc/gemm/gemm_api.h)."""
    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("D", c_void_p), ("D2", c_void_p), ("aux", c_void_p),
        ("M", c_int), ("N", c_int), ("K", c_int),
        ("lda", c_longlong), ("ldb", c_longlong), ("ldd", c_longlong), ("ldd2", c_longlong), ("ld_aux", c_longlong),
        ("a_rows", c_int), ("b_rows", c_int),
        ("d_cols", c_int), ("d2_cols", c_int), ("d_rows", c_int),
        ("a_mn", c_int), ("b_mn", c_int),
        ("epi", c_int), ("act", c_int),
        ("b_up_rows", c_int), ("d_up_cols", c_int),
        ("status", c_void_p),
        ("a_ready", c_void_p), ("a_ready_value", c_uint32), ("a_ready_rows", c_int), ("m_rotate", c_int),
        ("ag_src", c_void_p), ("ag_dst", c_void_p * MAX_RANKS), ("ag_flags", c_void_p * MAX_RANKS),
        ("ag_rows_per_rank", c_int), ("ag_ld", c_longlong),
        ("rank", c_int), ("world", c_int),
        ("rs_recv", c_void_p * MAX_RANKS), ("rs_count", c_void_p * MAX_RANKS),
        ("rs_expect", c_uint32), ("rs_out", c_void_p), ("rs_rows_per_rank", c_int),
        ("num_ctas", c_int), ("tile_n", c_int), ("pair", c_int),
        ("tiles", c_void_p), ("n_tiles_dev", c_void_p), ("max_tiles", c_int),
        ("d_done", c_void_p), ("k_ready", c_void_p), ("k_ready_value", c_uint32), ("k_ready_rows", c_int),
        ("b_scales", c_void_p), ("b_bits", c_int), ("pdl", c_int),
        ("ar_out", c_void_p * MAX_RANKS), ("ar_flag", c_void_p * MAX_RANKS), ("ar_expect", c_uint32),
        ("ag_split", c_int),
    ]


def available() -> bool:
    from . import _build
    return _build.lib_path().exists()


def checked() -> bool:
    """True when the loaded library is the checked build."""
    L = lib()
    return bool(L.mesh_checked_build())


def lib() -> ctypes.CDLL:
    """Load (building first if sources changed and nvcc is present) and return the library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from . import _build
        from .config import config
        check = bool(config().check)          # MESH_CHECK=1: the library with index / alignment checks in its kernels
        path = _build.lib_path(check)
        import os
        rebuild = os.environ.get("MESH_BUILD", "1") != "0"     # MESH_BUILD=0: load the library as it is, stale or not
        if not path.exists() or (rebuild and not _build.is_current(check) and _build.nvcc_path() is not None):
            try:
                path = _build.build(check=check)
            except Exception as e:  # keep a stale but loadable library usable
                if not path.exists():
                    raise RuntimeError(f"mesh_b200 native library is missing and could not be built: {e}") from e
        L = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
        L.mesh_last_error.restype = ctypes.c_char_p
        L.mesh_gemm_bf16.argtypes = [ctypes.POINTER(GemmArgs), c_void_p]
        L.mesh_gemm_bf16.restype = c_int
        _lib = L
        return L


def last_error() -> str:
    return lib().mesh_last_error().decode()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed (code {rc}): {last_error()}")
