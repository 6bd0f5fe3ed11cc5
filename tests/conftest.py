import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def port():
    from oracle import gwo
    return gwo.load("port")


@pytest.fixture(scope="session")
def checker():
    """The strongest CPU checker present: the reference's own code when its build exists, else the restatement."""
    from oracle import gwo
    return gwo.best()


@pytest.fixture(scope="session")
def ref():
    from oracle import gwo
    r = gwo.load("ref")
    if r is None:
        pytest.skip("oracle/_ref is not built (needs the reference sources)")
    return r
