import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Property tests run the same examples on every machine: a failure is then reproducible and a green run stays green.
try:
    from hypothesis import settings as _hsettings
    _hsettings.register_profile("repeatable", derandomize=True, deadline=None, database=None)
    _hsettings.load_profile("repeatable")
except ImportError:      # hypothesis is optional: tests/test_properties.py is skipped without it
    pass
