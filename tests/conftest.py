import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU and the built CUDA library")


@pytest.fixture(scope="session")
def backend():
    """The cuda backend; fails (never skips or falls back) when it cannot start."""
    from torchlette_b200 import backend as tb

    if not tb.initCuda(0):
        pytest.fail(f"cuda backend did not start: {tb.getCudaInitError()}")
    yield tb.getBackend()
    tb.destroyCuda()
