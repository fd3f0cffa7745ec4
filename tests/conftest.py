import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import katsu_ref

    katsu_ref.build()
    return katsu_ref


@pytest.fixture(scope="session")
def ctx():
    """One C-ABI context on device 0 for the whole GPU test session."""
    from katsu_b200 import cabi

    context = cabi.Context(0)
    yield context
    context.close()
