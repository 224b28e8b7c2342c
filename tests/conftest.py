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
    from oracle import born_oracle
    born_oracle.build()
    born_oracle.load()
    return born_oracle


@pytest.fixture(scope="session")
def lib():
    from born_b200 import build, _lib
    build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def sampler(lib):
    """A handle on cuda:0; GPU tests only.  Fails loudly when there is no device."""
    from born_b200 import Sampler
    s = Sampler(device=0, max_batch=1024, max_vocab=262144)
    yield s
    s.close()
