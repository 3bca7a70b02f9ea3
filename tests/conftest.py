"""Shared pytest setup: marker registration, import path, one build per session."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built_libraries():
    """Compile the native libraries and the oracle once (no-ops when up to date)."""
    from forward_b200 import build
    from oracle import eb_oracle

    build.build_all()
    eb_oracle.build()


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
