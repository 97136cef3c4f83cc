import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def deterministic_decode():
    """The tuned decode kernel with every SM kept to its own page range (the default), so that two launches on
    equal inputs can be compared bit for bit; set explicitly in case an earlier test left work stealing on."""
    from pie_b200 import ops

    ops.set_deterministic(True)
    yield
    ops.set_deterministic(False)
