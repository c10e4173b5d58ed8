import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built_oracle():
    """The oracle is compiled on first use; the reference build only where its tree is mounted."""
    from oracle import bindings
    if not os.path.exists(bindings.ORACLE_SO):
        bindings.build()
    yield
