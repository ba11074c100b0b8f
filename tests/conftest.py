"""pytest configuration: registers the ``gpu`` marker and makes the repository importable."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


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


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test, no kernel may have given up on a bounded wait."""
    yield
    if "gpu" in request.keywords:
        import torch
        if torch.cuda.is_available():
            from cai_b200.ops import device_status
            assert device_status(clear=True) == 0, "a kernel reported a wait timeout"
