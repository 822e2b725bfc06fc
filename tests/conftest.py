import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _guard_words(request):
    """After every GPU test: no kernel wrote past the end of a guarded device buffer (the step buffer, the
    cache groups, per-sequence state, sampler buffers, counters).  Buffers whose owner the test has dropped
    are held until this check has seen them."""
    if "gpu" not in request.keywords:
        yield
        return
    from llmoxide_b200 import guard

    guard.hold_until_checked(True)
    yield
    guard.check_all()
