"""Shared test plumbing: the `gpu` marker, import helpers and fixtures."""
import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PKG_NAME = "two-level-attention_b200"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def load_pkg(sub=None):
    """Import the package (its directory name is not a Python identifier)."""
    name = PKG_NAME if sub is None else f"{PKG_NAME}.{sub}"
    return importlib.import_module(name)


@pytest.fixture(scope="session")
def pkg():
    return load_pkg()


def golden(name):
    return np.load(os.path.join(GOLDEN, name))
