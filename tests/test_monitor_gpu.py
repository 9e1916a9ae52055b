"""Error monitor: cancels a bounded device wait past the running kernel, and notices a wait that ran out."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _wait_kernel(flag, limit_ns, st):
    from mesh_b200 import _native
    rc = _native.lib().mesh_wait_flag_test(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint32(1), ctypes.c_uint64(limit_ns),
                                           ctypes.c_void_p(st.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0


def test_monitor_cancels_and_reports():
    from mesh_b200.runtime.monitor import ErrorMonitor
    from mesh_b200.utils.status import MeshCanceled, MeshTimeout, check_status, clear_abort, status_block
    st = status_block()
    check_status()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    mon = ErrorMonitor(interval_ms=2)
    try:
        # a wait on a word nobody writes, limit 1.5 s: the host cancels it after 50 ms
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        _wait_kernel(flag, 1_500_000_000, st)
        time.sleep(0.05)
        mon.abort()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert dt < 1.0, dt
        with pytest.raises(MeshCanceled):
            check_status()
        mon.abort(False)
        time.sleep(0.02)
        clear_abort()
        mon.clear()
        torch.cuda.synchronize()
        # a wait that runs out by itself (50 ms) is seen by the monitor, which raises the abort word for everyone
        _wait_kernel(flag, 50_000_000, st)
        torch.cuda.synchronize()
        time.sleep(0.05)
        rep = mon.report()
        assert rep["seen_error"] and rep["code"] == "TIMEOUT" and rep["site"] == "host_flag" and rep["polls"] > 5, rep
        assert int(st[11].item()) == 1                       # abort spread to the watched block
        with pytest.raises(MeshTimeout):
            check_status()
        mon.clear()
        time.sleep(0.02)
        clear_abort()
        check_status()
        assert torch.ones(4, device="cuda").sum().item() == 4.0
    finally:
        mon.stop()
        clear_abort()
