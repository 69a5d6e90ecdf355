"""Helpers for the GPU parity tests: move NumPy arrays to the device, fetch results back."""
import numpy as np

import mytorch_b200 as mt
from mytorch_b200.backends.backend_dispatcher import BackendDispatcher

DEV = "cuda:0"


def dev(a, grad=False):
    a = np.ascontiguousarray(a)
    return mt.tensor(a, device=DEV, requires_grad=grad and a.dtype.kind == "f")


def host(t):
    return None if t is None else t.to("cpu")._numpy()


def op(name):
    return BackendDispatcher.instance().dispatch("cuda", name)
