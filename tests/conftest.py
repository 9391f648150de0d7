import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(autouse=True)
def _device_status_is_clean(request):
    """After every GPU test: no kernel of the library gave up a device-side wait (the status word of the last call)."""
    yield
    if "gpu" not in request.keywords:
        return
    try:
        import torch
        if not torch.cuda.is_available():
            return
        import flamia_blackwell_attention_b200 as F
    except Exception:
        return
    F.check_status()
