"""Shared test setup: import paths, the `gpu` marker, and small tensor helpers."""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
PACKAGE_DIR = ROOT / "robotics-the-speedup-paradox_b200"
for entry in (str(ROOT), str(PACKAGE_DIR)):
    if entry not in sys.path:
        sys.path.insert(0, entry)

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_cuda = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_cuda = False
    if has_cuda:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN / "integer_golden.npz")


def bf16_from_bits(bits):
    """uint16 bit patterns -> float32 values."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
