"""Shared fixtures.  ``gpu`` marks tests that need a CUDA device and the native library."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    """Outputs of the reference's own CPU code (tests/golden/make_golden.py)."""

    return dict(np.load(ROOT / "tests" / "golden" / "reference_vectors.npz"))
