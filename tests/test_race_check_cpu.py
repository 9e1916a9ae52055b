"""The host runtime under ThreadSanitizer: service thread, counters, stats readers, host engine and the engine bridge
used from several threads at once (``mesh_b200/csrc/standalone/race_check.cpp``)."""
import pytest


def test_host_runtime_has_no_data_race_under_thread_sanitizer():
    from mesh_b200 import _build
    rc, text = _build.run_race_check()
    if rc == -1:
        pytest.skip(text)
    assert rc == 0, text
    assert "ThreadSanitizer" not in text, text
    assert "race_check: ok" in text
