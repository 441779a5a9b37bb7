import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def orc():
    """The oracle bindings module (oracle/oracle.py)."""
    m = entry.load_oracle()
    if not os.path.exists(m.ORACLE_SO):
        m.build(ref=False)
    return m


@pytest.fixture(scope="session")
def oracle(orc):
    return orc.Oracle()


@pytest.fixture(scope="session")
def pkg():
    """The product package; building is part of loading it here so the CPU suite needs no separate step."""
    p = entry.load_package()
    if not os.path.exists(p.LIB_PATH):
        import subprocess
        subprocess.check_call([sys.executable, os.path.join(entry.PKG_DIR, "build.py")])
    p.lib()
    return p
