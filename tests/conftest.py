"""Shared pytest set-up: markers, import paths and fixture loading."""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "transformers-turboquant_b200")
for p in (ROOT, PKG_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box only)")


def load_golden(name: str):
    return np.load(os.path.join(GOLDEN_DIR, name))


@pytest.fixture(scope="session")
def golden_constants():
    return load_golden("constants.npz")


@pytest.fixture(scope="session")
def golden_wire():
    return load_golden("wire_format.npz")


@pytest.fixture(scope="session")
def golden_comp():
    return load_golden("compressors.npz")


@pytest.fixture(scope="session")
def golden_family():
    return load_golden("family_gpt2.npz")
