"""The checked build (``MESH_CHECK=1``: the library compiled with index / alignment checks inside its kernels).

Small-shape tests of the kernels run against it in a child process, and a tile descriptor that names rows outside
its matrix is recorded as BOUNDS in the status block, with the kernel returning normally, instead of being issued.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, timeout=900):
    env = dict(os.environ, MESH_CHECK="1")
    return subprocess.run([sys.executable, *args], cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def test_small_shapes_pass_under_the_checked_build():
    r = _run(["-m", "pytest", "-q", "-x", "-m", "gpu", "tests/test_gemm_gpu.py", "tests/test_moe_gpu.py",
              "tests/test_ops_gpu.py", "tests/test_tp_ffn_gpu.py", "-k", "not multi", "-p", "no:cacheprovider"])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


_BAD_TILE = r'''
import ctypes, torch
from mesh_b200 import _native
from mesh_b200.utils.status import MeshDeviceError, check_status, status_block
assert _native.checked(), "MESH_CHECK=1 must load the checked library"
dev = torch.device("cuda", 0)
a = torch.randn(512, 256, device=dev).bfloat16()
b = torch.randn(256, 256, device=dev).bfloat16()
out = torch.zeros(512, 256, device=dev).bfloat16()
# one good tile and one whose first row lies far outside A
tiles = torch.tensor([[0, 0, 4, 0, 0, 0, 0, 0], [10_000_000, 0, 4, 0, 0, 256, 0, 0]], dtype=torch.int32, device=dev)
n = torch.tensor([2], dtype=torch.int32, device=dev)
g = _native.GemmArgs()
g.A, g.B, g.D = a.data_ptr(), b.data_ptr(), out.data_ptr()
g.M, g.N, g.K = 512, 256, 256
g.lda, g.ldb, g.ldd = 256, 256, 256
g.a_rows, g.b_rows, g.d_cols, g.d_rows = 512, 256, 256, 512
g.status = status_block(dev).data_ptr()
g.world, g.pair = 1, 1
g.tiles, g.n_tiles_dev, g.max_tiles = tiles.data_ptr(), n.data_ptr(), 2
rc = _native.lib().mesh_gemm_bf16(ctypes.byref(g), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
assert rc == 0, _native.last_error()
try:
    check_status()
    raise SystemExit("the bad tile was not reported")
except MeshDeviceError as e:
    assert e.record["code"] == "BOUNDS" and e.record["site"] == "check" and e.record["seen"] == 10_000_000, e.record
check_status()                                   # cleared; the context still answers
assert float(torch.ones(8, device=dev).sum()) == 8.0
print("ok")
'''


def test_bad_tile_descriptor_is_recorded_not_issued():
    r = _run(["-c", _BAD_TILE], timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
