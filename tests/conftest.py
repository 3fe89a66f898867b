import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def fkb_lib():
    """The C-ABI library, built in-tree if missing or stale."""
    from fusedkernellibrary_b200 import abi, build
    build.build()
    return abi.load_library()


@pytest.fixture(scope="session")
def oracle_port():
    from oracle import port
    port.build()
    return port
