import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def lib_built():
    """Build (or find) libb200cp.so; the CPU suite only loads it and checks its exports."""
    from paralleltnnlayers_b200 import build
    return build.build()
