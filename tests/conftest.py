"""Shared pytest configuration.

Markers: ``gpu`` marks every test that needs a CUDA device; everything else runs on CPU.
The product package lives in ``llm_quantization-kernel_b200/`` (importable as
``crispybits_kernels`` once that directory is on ``sys.path``); the CPU oracle lives in
``oracle/`` and is imported by tests only.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "llm_quantization-kernel_b200")
for p in (ROOT, PKG, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """The committed fixtures produced by tests/golden/make_golden.py from the reference."""
    path = os.path.join(ROOT, "tests", "golden", "golden_v1.npz")
    return np.load(path, allow_pickle=False)
