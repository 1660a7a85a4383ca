import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _collect_dead_engines():
    """Engines own captured CUDA graphs.  One that a finished test left in a reference cycle (a traceback frame, a
    future) would otherwise be destroyed by whichever allocation triggers the collector — possibly in the middle of
    another test's graph capture, where destroying a graph is not permitted.  Collect at the test boundary instead."""
    yield
    import gc

    gc.collect()
