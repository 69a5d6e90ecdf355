"""Host-side storage operations for tensors that live on ``device="cpu"``.

Models are usually built on the CPU (seeded initialisation) and then moved with ``.to("cuda")``,
and checkpoints travel through CPU tensors, so fill / random init / copy / cast / reshape must
work there.  Nothing else is registered: arithmetic on CPU tensors raises, by design — this
package has no CPU compute backend.

Random fills restate ``mytorch/backends/cpu/ops/elementwise_ops.py:11-22`` (seed NumPy's
global generator with the per-tensor seed, then draw), so that a model initialised here under
``manual_seed(s)`` has bit-identical weights to the reference initialised on its CPU backend.
"""
import numpy as np

from mytorch_b200.backends.backend_dispatcher import BackendDispatcher
from mytorch_b200.backends.utils import calculate_reshaped_shape

_reg = BackendDispatcher.instance().register_backend_function


@_reg("cpu", "fill")
def cpu_fill(x, value):
    np.copyto(x._numpy(), value)


@_reg("cpu", "normal")
def cpu_normal(x, seed, mean, stddev):
    np.random.seed(seed)
    x._cpu_array = np.random.normal(mean, stddev, x.shape).astype(x.dtype.np_dtype)


@_reg("cpu", "uniform")
def cpu_uniform(x, seed, a, b):
    np.random.seed(seed)
    x._cpu_array = np.random.uniform(low=a, high=b, size=x.shape).astype(x.dtype.np_dtype)


@_reg("cpu", "copy")
def cpu_copy(x, y):
    np.copyto(x._numpy(), y._numpy())


@_reg("cpu", "cast")
def cpu_cast(x, dtype):
    from mytorch_b200.tensor import Tensor

    return Tensor(cpu_array=x._numpy().astype(dtype.np_dtype), dtype=dtype, device=x.device)


@_reg("cpu", "reshape")
def cpu_reshape(x, shape):
    from mytorch_b200.tensor import Tensor

    out = Tensor(tensor=x)
    out.shape = calculate_reshaped_shape(x.shape, shape)
    out._cpu_array = x._numpy().reshape(out.shape)
    return out
