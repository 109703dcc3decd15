"""Shared fixtures.  Tests that need a GPU carry `@pytest.mark.gpu`; everything else runs on CPU."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "w8a8_golden.npz")


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library (built on demand when nvcc is present)."""
    from braid_b200 import _lib, build
    if build.is_stale():
        build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def Q(lib):
    """`braid_b200.quant` with the kernels warmed (GPU sessions only)."""
    from braid_b200 import quant
    if torch.cuda.is_available():
        quant.warm_fused(True)
    return quant
