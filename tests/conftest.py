import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")
    # pytest-timeout registers this itself; without the plugin the mark is inert instead of unknown
    config.addinivalue_line("markers", "timeout(seconds): per-test time limit (pytest-timeout)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# GPU tests run with guard bands around the package's workspaces, caches and symmetric buffers (utils/canary.py): no
# device memory checker can be run on the test hosts, so an overrun is caught by the bytes next to the buffer.
os.environ.setdefault("B200_CANARY", "1")


@pytest.fixture(autouse=True)
def _guard_bands_intact(request):
    yield
    if "gpu" not in request.keywords:
        return
    from deepseek_v4_2080ti_b200.utils import canary
    if canary.is_enabled() and canary.live_buffers():
        canary.assert_clean()
