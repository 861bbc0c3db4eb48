"""Shared pytest configuration: markers and import path."""
import os
import sys

import pytest

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _canary_pads_intact(request):
    """With ``MSRL_DEBUG_CANARY=1`` every GPU test ends with a check that no kernel wrote outside the
    outputs the ops allocated for it."""
    yield
    if "gpu" in request.keywords and os.environ.get("MSRL_DEBUG_CANARY") == "1":
        from mindspeed_rl_b200.ops import guard

        guard.check(request.node.name)
