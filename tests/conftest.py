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


def rel_l2(a, b):
    """||a-b||_2 / ||b||_2 — used for whole-model gradients.  A pre-activation that is within
    rounding distance of 0 can fall on different sides of a ReLU in two correct implementations;
    the gradient at that one element then differs by its full magnitude, so a max-norm comparison
    of activation or weight gradients through many ReLU layers is ill-conditioned while the L2
    error stays of the order sqrt(fraction of flipped elements)."""
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    return float(np.linalg.norm(a - b) / max(float(np.linalg.norm(b)), 1e-30))


def summarize(arr, sample=64):
    a = np.asarray(arr, dtype=np.float64).reshape(-1)
    idx = np.linspace(0, a.size - 1, min(sample, a.size)).astype(np.int64)
    return np.array([a.sum(), np.abs(a).sum(), np.sqrt((a * a).sum())]), a[idx]


@pytest.fixture(scope="session")
def golden():
    return load_golden


@pytest.fixture(autouse=True, scope="module")
def tensor_core_kernels_never_gave_up():
    """Every bounded wait inside the tensor-core kernels gives up after its limit and records a code
    in a status word instead of hanging; a module of GPU tests must end with that word still clear."""
    yield
    from mytorch_b200.backends.cuda.env import CudaEnv

    if CudaEnv._instance is not None:
        assert CudaEnv._instance.tensor_core_status() == 0
