"""Test configuration: the ``gpu`` marker, import paths, shared helpers.

``-m "not gpu"`` covers the oracle against the golden vectors, the host logic and the
C ABI surface (no compute calls); ``-m gpu`` holds the parity tests proper, which call
the CUDA kernels through the C ABI and compare with the CPU oracle.
"""
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
PKG = REPO / "writes-that-matter_b200"
for p in (str(PKG), str(REPO)):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def native_lib():
    """The built shared library (compiled on demand: nvcc cross-compiles without a GPU)."""
    from lcgemm import _native

    _native.build()
    return _native.lib()


def bf16_from_bits(arr):
    import numpy as np
    import torch

    return torch.from_numpy(np.ascontiguousarray(arr)).view(torch.bfloat16)
