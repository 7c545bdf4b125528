import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped, not failed, where no device exists."""
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_small():
    import torch
    return torch.load(os.path.join(GOLDEN, "reference_small.pt"), weights_only=False)


@pytest.fixture(scope="session")
def golden_paged():
    import torch
    return torch.load(os.path.join(GOLDEN, "reference_paged.pt"), weights_only=False)


@pytest.fixture(scope="session")
def golden_mla_paged():
    import torch
    return torch.load(os.path.join(GOLDEN, "reference_mla_paged.pt"), weights_only=False)
