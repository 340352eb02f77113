import os
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as entry

    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle import build as oracle_build
    from oracle import oracle as o

    oracle_build.build_oracle()
    return o
