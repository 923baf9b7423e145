import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle import moe_oracle
    moe_oracle.build()
    return moe_oracle


@pytest.fixture(scope="session")
def mc(pkg):
    return pkg.moe_cuda


@pytest.fixture(scope="session")
def synth(pkg):
    return pkg.synth


@pytest.fixture()
def ctx(mc):
    """A fresh context on cuda:0; fails (never skips) if the CUDA path is unusable."""
    c = mc.Ctx(0)
    c.check()
    yield c
    c.close()
