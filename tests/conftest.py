import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built():
    """Builds (or reuses) the cubin and libiree_b200.so; the oracle libraries too."""
    from iree_b200 import build
    import oracle
    build.build_all()
    oracle.build()
    return True


@pytest.fixture(scope="session")
def ctx(built):
    import iree_b200
    c = iree_b200.Context(0)
    yield c
    c.close()
