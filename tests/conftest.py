"""pytest configuration: the `gpu` marker and shared seeded generators."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    """A `gpu` test on a machine without a device is skipped rather than failed, so that a plain
    `pytest tests/` works on a CPU box; `-m gpu` on a GPU box runs them all."""
    try:
        import torch
        has = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has = False
    if has:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def rng():
    return np.random.default_rng(20261125)
