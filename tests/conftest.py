import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "slow: larger parity cases")


@pytest.fixture(scope="session")
def mk():
    """The product package (ctypes over libmacllm_b200.so)."""
    entry.ensure_built()
    return pkg


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle's math library."""
    from oracle import mathlib
    mathlib.build()
    return mathlib
