import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the built sm_100a library")


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
def _reset_batch_invariant_mode():
    """Speculative-decoding tests switch the projection kernels to their batch-invariant mode process-wide; later tests
    start from the default again."""
    yield
    try:
        from grimoire_b200.ops import linear

        linear.set_batch_invariant(False)
    except Exception:
        pass
