import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as module

    module.build()
    return module


@pytest.fixture(scope="session")
def runtime():
    """One native runtime per test session. No fallback: fails if the library or GPU is missing."""
    from llmopt_b200 import cuda_native

    return cuda_native.Runtime()


def f16_bits(values):
    return np.array(values, dtype=np.uint16).view(np.float16)


def assert_close_f16(actual, expected, rel=2e-3, label=""):
    """max |a - e| <= rel * max(|e|_inf, tiny): the reference's parity bound for
    fp16 outputs with fp32 accumulation (relative to the output scale)."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape, f"{label}: shape {actual.shape} != {expected.shape}"
    assert np.all(np.isfinite(actual)), f"{label}: non-finite output"
    scale = max(np.max(np.abs(expected)), 1e-6)
    error = np.max(np.abs(actual - expected)) / scale
    assert error <= rel, f"{label}: max error {error:.3e} of output scale exceeds {rel:.1e}"
    return error
