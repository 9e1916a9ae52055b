import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (sm_100a); run with -m gpu on a B200")
    config.addinivalue_line("markers", "multigpu: needs at least 2 GPUs")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        # Every GPU test gets a time limit (multi-rank tests spawn child processes that wait on each other): a test
        # that cannot finish fails after a few minutes instead of holding the run.  The marker needs the
        # pytest-timeout plugin; without it, it is inert.
        for item in items:
            if "gpu" in item.keywords and item.get_closest_marker("timeout") is None:
                item.add_marker(pytest.mark.timeout(420))
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multigpu" in item.keywords:
            item.add_marker(skip)
