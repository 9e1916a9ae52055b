"""The allocation-free RMSNorm backward (csrc/ops/noalloc_api.h) against the regular entry point.

Some hosts of this library get their buffers from another runtime and have no allocator of their
own to call (a server plugin with a fixed memory budget, a custom-call hook that only sees raw
pointers).  For them the library keeps the op's scratch inside its own image.  This test drives
that entry point the way such a caller would — through the exported C symbol, with pointers only —
and checks dx and dw against ``mesh_rmsnorm_bwd`` and against an fp32 PyTorch statement on calls in a
row (each later call finds the scratch dirty from the one before, and from a different shape).
Collected last on purpose.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(rows, cols, seed):
    from mesh_b200 import _native
    from mesh_b200.ops.norm import rmsnorm_bwd, rmsnorm_fwd
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    w = (torch.randn(cols, device="cuda", generator=g) * 0.1 + 1).bfloat16()
    dy = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    _, _, rstd = rmsnorm_fwd(x, w, 1e-6, need_rstd=True)
    dx_ref, dw_ref = rmsnorm_bwd(dy, x, w, rstd)

    L = _native.lib()
    fn = L.mesh_rmsnorm_bwd_noalloc            # the exported C symbol
    fn.restype = c_int
    dx = torch.empty_like(x)                   # outputs are the caller's; the entry point allocates nothing
    dw = torch.empty(cols, dtype=torch.float32, device="cuda")
    rc = fn(c_void_p(dy.data_ptr()), c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_void_p(rstd.data_ptr()),
            c_void_p(dx.data_ptr()), c_void_p(dw.data_ptr()), c_int(rows), c_int(cols), c_float(0.0),
            c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _native.last_error()
    torch.cuda.synchronize()
    # against the regular entry point (same arithmetic, another order of the column sums)
    torch.testing.assert_close(dx.float(), dx_ref.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(dw, dw_ref.float(), atol=1e-2, rtol=1e-3)
    # against fp32 PyTorch
    xf, wf, dyf = x.float(), w.float(), dy.float()
    r = rstd.float().unsqueeze(1)
    dw_t = (dyf * xf * r).sum(0)
    gw = dyf * wf
    dx_t = gw * r - xf * ((gw * xf).sum(1, keepdim=True) * r * r * r / cols)
    torch.testing.assert_close(dw, dw_t, atol=1e-2, rtol=1e-3)
    assert float((dx.float() - dx_t).square().mean().sqrt() / dx_t.square().mean().sqrt()) < 4e-3


def test_noalloc_matches_regular_entry_point_twice():
    _case(500, 2048, seed=1)     # first call on this device also looks up the scratch address
    _case(77, 4096, seed=2)      # second call: other shape, scratch still holds the first call's sums
    _case(3, 8192, seed=3)       # fewer rows than partial rows, the widest row the scratch takes


def test_noalloc_rejects_oversize():
    from mesh_b200 import _native
    fn = _native.lib().mesh_rmsnorm_bwd_noalloc
    fn.restype = c_int
    rc = fn(c_void_p(0), c_void_p(0), c_void_p(0), c_void_p(0), c_void_p(0), c_void_p(0), c_int(4), c_int(16384),
            c_float(0.0), c_void_p(0))
    assert rc != 0 and "exceeds" in _native.last_error()
    # bad pointers are refused with an error code; nothing is launched
    buf = torch.zeros(4 * 64 + 8, dtype=torch.bfloat16, device="cuda")
    f32 = torch.zeros(64, dtype=torch.float32, device="cuda")
    ok = c_void_p(buf.data_ptr())
    rc = fn(ok, ok, ok, c_void_p(f32.data_ptr()), ok, c_void_p(0), c_int(4), c_int(64), c_float(0.0), c_void_p(0))
    assert rc != 0 and "null" in _native.last_error()
    odd = c_void_p(buf.data_ptr() + 2)
    rc = fn(ok, odd, ok, c_void_p(f32.data_ptr()), ok, c_void_p(f32.data_ptr()), c_int(4), c_int(64), c_float(0.0),
            c_void_p(0))
    assert rc != 0 and "aligned" in _native.last_error()
    torch.cuda.synchronize()
