import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")


@pytest.fixture(scope="session")
def cuda_engine():
    """The 'cuda' backend on device 0; fails loudly if it cannot be created."""
    import tfjs_b200
    tfjs_b200.ENGINE.set_backend("cuda")
    tfjs_b200.ENGINE.is_test = True
    return tfjs_b200.ENGINE
