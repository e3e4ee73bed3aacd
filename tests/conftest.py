import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    """GPU tests skip themselves cleanly when no GPU is visible (e.g. a bare `pytest tests/`)."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA GPU visible")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def option():
    """Sets tuning options of the library for one test (ternix_b200_set_option) and restores the defaults after it."""
    import ternixengine_b200 as tb
    touched = []

    def set_option(name, value):
        tb.set_option(name, value)
        touched.append(name)

    yield set_option
    for name in touched:
        tb.set_option(name, None)
