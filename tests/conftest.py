"""Shared test configuration: the `gpu` marker, import paths and fixture loading."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "fp8-compatibility-layer_b200")
for p in (PKG, ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "tfp8_golden.npz"))


@pytest.fixture(scope="session")
def golden_c1():
    return np.load(os.path.join(ROOT, "tests", "golden", "config1_golden.npz"))
