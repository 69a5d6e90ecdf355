import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def rel_err(a, b):
    """max |a-b| / max |b| — the 'relative' error all parity tolerances are quoted in."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.max(np.abs(a - b)) / max(float(np.max(np.abs(b))), 1e-30))


def summarize(arr, sample=64):
    a = np.asarray(arr, dtype=np.float64).reshape(-1)
    idx = np.linspace(0, a.size - 1, min(sample, a.size)).astype(np.int64)
    return np.array([a.sum(), np.abs(a).sum(), np.sqrt((a * a).sum())]), a[idx]


@pytest.fixture(scope="session")
def golden():
    return load_golden
