"""Shared pytest set-up: the `gpu` marker, import paths, and the `sk` fixture.

Tests marked `gpu` are the parity tests proper: they call the CUDA library through its C-ABI
and compare with the CPU oracle. Everything else runs without a GPU.
"""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_PY = os.path.join(ROOT, "5090-blackwell-kernels_b200", "python")
for p in (ROOT, PKG_PY):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(ROOT, "tests", "golden", f"{name}.npz"))

    return load


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle

    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def sk():
    """The product package on a CUDA device. A missing extension or device is an error for a
    gpu test, never a skip to a fallback."""
    import torch

    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    import spark_kernels

    return spark_kernels
