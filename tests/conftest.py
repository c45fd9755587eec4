import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))      # orc.py, the numpy binding of the CPU oracle


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu")


@pytest.fixture(scope="session")
def dev():
    """The library with device 0 selected; a GPU test fails (not skips) when that cannot be done."""
    import ufsm_b200
    L = ufsm_b200.lib()
    rc = L.nn_init(0)
    assert rc == 0, "nn_init(0) failed: %s" % (L.lp_check() or b"").decode()
    return L
