"""Shared test plumbing: the `gpu` marker, import paths for the oracle (test-only) and the package."""
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
ORACLE_DIR = os.path.join(ROOT, "oracle")
if ORACLE_DIR not in sys.path:
    sys.path.insert(0, ORACLE_DIR)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    import kda_oracle

    kda_oracle.build()
    return kda_oracle


@pytest.fixture(scope="session")
def pkg():
    """The package; its directory name carries a hyphen, so it is imported by name."""
    return importlib.import_module("glm53f-afd_b200")
