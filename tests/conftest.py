"""Shared pytest configuration: the ``gpu`` marker and golden-vector loading."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Vectors produced by the DIMQ reference (tests/golden/make_golden.py)."""
    with np.load(ROOT / "tests" / "golden" / "reference_vectors.npz") as data:
        return {k: data[k] for k in data.files}


@pytest.fixture(scope="session")
def cuda_device():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
