import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_sessionstart(session):
    """Build the native library, the host extension and the oracle if they are not there yet."""
    from flashrwkv_b200 import build as native

    native.build_all()
    from tests.native import build_probe

    build_probe.build()


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure); built on first use."""
    from oracle import wkv7_oracle

    wkv7_oracle.build()
    return wkv7_oracle
