import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def kd():
    """The product package (loads libkdnn_b200.so; builds it first if stale)."""
    import __graft_entry__ as ge
    ge.build()
    return ge.load_package()


@pytest.fixture(scope="session")
def port():
    from oracle import oracle as O
    O.build()
    return O.Port()


@pytest.fixture(scope="session")
def ref():
    """The reference's own operators; skipped when oracle/_ref was never built."""
    from oracle import oracle as O
    if not O.Ref.available():
        pytest.skip("oracle/_ref/libkdnn_ref.so not present")
    return O.Ref()
