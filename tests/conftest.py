"""Shared fixtures.  GPU tests carry the ``gpu`` marker; everything else runs on CPU."""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(GOLDEN_DIR, "nvfp4_golden.npz"))


@pytest.fixture(scope="session")
def golden_large():
    with open(os.path.join(GOLDEN_DIR, "nvfp4_golden_large.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.build()
    return o


def golden_case_names() -> list[str]:
    return [str(n) for n in np.load(os.path.join(GOLDEN_DIR, "nvfp4_golden.npz"))["names"]]
