"""pytest configuration: the ``gpu`` marker and import path."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "slow: long-running variant of a test that has a fast form (deselect with -m 'not slow')")


def pytest_collection_modifyitems(config, items):
    import torch

    if not os.environ.get("LETHE_RUN_SLOW"):
        slow = pytest.mark.skip(reason="slow variant: set LETHE_RUN_SLOW=1 to run it")
        for it in items:
            if "slow" in it.keywords:
                it.add_marker(slow)

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)
