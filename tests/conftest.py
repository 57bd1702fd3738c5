"""Shared test setup: the gpu marker, the tiny configurations, model folders."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (a B200)")
    # The plain implementation is the tests' yardstick, so its float32 results must
    # not depend on how a library splits work over host threads.  Seen with 16
    # threads: the first attention product of a process was off by 3e-5 in a block of
    # rows about once in six processes (and right when computed again); never with one
    # thread.  The tiny models need no more.
    import torch
    torch.set_num_threads(1)


def pytest_collection_modifyitems(config, items):
    import torch
    # a watchdog on every test (as the reference's tests have one,
    # tests/test_attention.c:343): a test that hangs ends the run with the stacks of
    # all threads instead of holding the machine.  Only where the plugin is there.
    if config.pluginmanager.hasplugin("timeout"):
        for item in items:
            if item.get_closest_marker("timeout") is None:
                item.add_marker(pytest.mark.timeout(600, method="thread"))
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
