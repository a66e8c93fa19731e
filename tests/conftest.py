import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle_port():
    from oracle import oracle
    return oracle.load("port")


@pytest.fixture(scope="session")
def oracle_ref():
    from oracle import oracle
    if not oracle.available("reference"):
        try:
            oracle.build("reference")
        except Exception:
            pass
    if not oracle.available("reference"):
        pytest.skip("oracle/_ref/libogle_ref.so not built (reference tree absent)")
    return oracle.load("reference")
