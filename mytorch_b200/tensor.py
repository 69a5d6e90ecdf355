"""Tensor and Device.  API of the reference's ``mytorch/tensor.py:52-394`` (constructor keywords,
``tensor()`` factory, ``to`` / ``item`` / ``detach`` / ``numpy`` rules, operator overloads,
``backward``), with one storage difference that user code cannot observe: a 4-D float32
tensor on a CUDA device is stored channels-last (N,H,W,C) because that is what the TMA /
tensor-core kernels read.  ``shape`` stays logical NCHW and every host transfer converts.
"""
from __future__ import annotations

import math
import numbers
from typing import Optional

import numpy as np

from mytorch_b200.autograd import DAGTracker
from mytorch_b200.backends.backend_dispatcher import BackendDispatcher
from mytorch_b200.dtype import DType, float32


class InvalidDeviceError(RuntimeError):
    def __init__(self, device_type):
        super().__init__(f"Invalid device type: {device_type}")


class InvalidDataTypeError(RuntimeError):
    def __init__(self, data_type):
        super().__init__(f"Invalid data type: {data_type}")


class InvalidShapeError(RuntimeError):
    def __init__(self, shape):
        super().__init__(f"Invalid tensor shape: {shape}")


class MismatchDevicesError(RuntimeError):
    def __init__(self, device_types):
        super().__init__(f"Mismatch devices between tensors: {device_types}")


class MismatchDataTypesError(RuntimeError):
    def __init__(self, data_types):
        super().__init__(f"Mismatch data types between tensors: {data_types}")


class MismatchShapesError(RuntimeError):
    def __init__(self, shapes):
        super().__init__(f"Mismatch shapes between tensors: {shapes}")


def shape_size(shape):
    return math.prod(shape)


class Device:
    """``"cpu"``, ``"cuda"`` or ``"cuda:<index>"`` (mytorch/tensor.py:52-81)."""

    def __init__(self, device):
        if isinstance(device, Device):
            self.type, self.index = device.type, device.index
            return
        text = device.strip()
        head, sep, tail = text.partition(":")
        self.type = head.strip()
        self.index = int(tail) if sep else None

    def __eq__(self, other):
        return isinstance(other, Device) and self.type == other.type and self.index == other.index

    def __hash__(self):
        return hash((self.type, self.index))

    def __repr__(self):
        return self.type if self.index is None else f"{self.type}:{self.index}"


def _dispatch(device_type, name):
    return BackendDispatcher.instance().dispatch(device_type, name)


def channels_last(shape, dtype, device_type):
    """Storage rule: 4-D float32 device tensors are physically (N,H,W,C)."""
    return device_type == "cuda" and len(shape) == 4 and dtype is float32


def tensor(data, dtype=None, device=None, requires_grad=False):
    data = np.array(data)
    if dtype is not None:
        data = data.astype(dtype.np_dtype)
    return Tensor(cpu_array=data, dtype=dtype, device=device, requires_grad=requires_grad)


class Tensor:
    def __init__(self, cpu_array=None, dtype: Optional[DType] = None, shape=None, device=None,
                 tensor: Optional["Tensor"] = None, requires_grad: bool = False):
        self.requires_grad = requires_grad
        self.grad = None
        self._grad_node = None

        if tensor is not None:  # alias: shares storage with `tensor`
            self._cpu_array = tensor._cpu_array
            self._native_array = tensor._native_array
            self.dtype, self.shape, self.device = tensor.dtype, tensor.shape, tensor.device
            self._nhwc = tensor._nhwc
            return

        self.device = Device(device if device is not None else "cpu")
        if self.device.type not in ("cpu", "cuda"):
            raise InvalidDeviceError(self.device.type)

        if dtype is not None:
            if not isinstance(dtype, DType):
                raise InvalidDataTypeError(dtype)
            self.dtype = dtype
            if cpu_array is not None and np.dtype(dtype.np_dtype) != cpu_array.dtype:
                raise InvalidDataTypeError(dtype)
        elif cpu_array is not None:
            self.dtype = DType.from_np_dtype(cpu_array.dtype)
        else:
            raise InvalidDataTypeError(dtype)

        if shape is not None:
            self.shape = tuple(int(s) for s in shape)
            if cpu_array is not None and self.shape != cpu_array.shape:
                raise InvalidShapeError(self.shape)
        elif cpu_array is not None:
            self.shape = tuple(cpu_array.shape)
        else:
            raise InvalidShapeError(shape)

        self._cpu_array = None
        self._native_array = None
        self._nhwc = channels_last(self.shape, self.dtype, self.device.type)

        if self.device.type == "cpu":
            self._cpu_array = cpu_array if cpu_array is not None else np.zeros(self.shape, dtype=self.dtype.np_dtype)
        else:
            nbytes = self.dtype.itemsize() * shape_size(self.shape)
            self._native_array = _dispatch("cuda", "allocate_memory")(self.device.index, nbytes)
            if cpu_array is not None:
                _dispatch("cuda", "upload")(self, cpu_array)

        if self.requires_grad and not self.dtype.is_floating:
            raise RuntimeError(f"tensor of type {self.dtype} cannot require gradient")

    # ------------------------------------------------------------------ movement
    def _to_device(self, device):
        device = Device(device)
        if self.device == device:
            return self
        if self.device.type == "cpu":
            return Tensor(cpu_array=self._cpu_array, device=device, requires_grad=self.requires_grad)
        if device.type == "cpu":
            return Tensor(cpu_array=_dispatch("cuda", "download")(self), device="cpu", requires_grad=self.requires_grad)
        out = Tensor(dtype=self.dtype, shape=self.shape, device=device, requires_grad=self.requires_grad)
        _dispatch("cuda", "transfer_memory")(out._native_array, self._native_array)
        return out

    def _to_dtype(self, dtype):
        from mytorch_b200.ops.cast import _cast

        return _cast(self, dtype)

    def to(self, device=None, dtype=None):
        return self._to_device(self.device if device is None else device)._to_dtype(self.dtype if dtype is None else dtype)

    def _host_array(self):
        return self._cpu_array if self.device.type == "cpu" else _dispatch("cuda", "download")(self)

    def __repr__(self):
        text = np.array2string(self._host_array(), threshold=50, separator=", ")
        return f'tensor({text}, dtype={self.dtype}, device="{self.device}")'

    def item(self):
        return self._host_array().item()

    def detach(self):
        return Tensor(tensor=self, requires_grad=False)

    def numpy(self):
        if self.requires_grad:
            raise RuntimeError("Tensor that requires gradient cannot be converted to NumPy array")
        return self._numpy()

    def _numpy(self):
        if self._cpu_array is None:
            raise RuntimeError("Tensor that not on CPU cannot be converted to numpy")
        return self._cpu_array

    def _native(self):
        if self._native_array is None:
            raise RuntimeError("Tensor does not have native array")
        return self._native_array

    # ------------------------------------------------------------------ in-place
    def fill_(self, value):
        from mytorch_b200.ops.elementwise_ops import _fill

        _fill(self, value)

    def copy_(self, tensor):
        from mytorch_b200.ops.broadcast_binary_ops import _copy

        if not isinstance(tensor, Tensor) or self.dtype != tensor.dtype:
            raise RuntimeError(f"Invalid tensor type to copy from: {tensor}")
        _copy(self, tensor.to(self.device))

    def normal_(self, mean, std):
        from mytorch_b200.ops.elementwise_ops import _normal
        from mytorch_b200.rand_generator import RandGenerator

        _normal(self, RandGenerator.instance().generate(), mean, std)

    def uniform_(self, a, b):
        from mytorch_b200.ops.elementwise_ops import _uniform
        from mytorch_b200.rand_generator import RandGenerator

        _uniform(self, RandGenerator.instance().generate(), a, b)

    # ------------------------------------------------------------------ math
    def sum(self, dim=None, keepdim=False):
        from mytorch_b200.ops.reduce_ops import sum as func

        return func(self, dim, keepdim)

    def mean(self, dim=None, keepdim=False):
        from mytorch_b200.ops.reduce_ops import mean as func

        return func(self, dim, keepdim)

    def reshape(self, shape):
        from mytorch_b200.ops.basic_ops import reshape as func

        return func(self, shape)

    def permute(self, dims):
        from mytorch_b200.ops.basic_ops import permute as func

        return func(self, dims)

    def _cast_other_to_tensor(self, other):
        if isinstance(other, Tensor):
            return other
        if isinstance(other, numbers.Number):
            return Tensor(cpu_array=np.array(other, dtype=self.dtype.np_dtype), device=self.device)
        if isinstance(other, np.ndarray):
            return Tensor(cpu_array=other.astype(self.dtype.np_dtype), device=self.device)
        raise InvalidDataTypeError(type(other))

    def _binary(self, name, other, reverse=False, *extra):
        import mytorch_b200.ops.broadcast_binary_ops as B

        other = self._cast_other_to_tensor(other)
        a, b = (other, self) if reverse else (self, other)
        return getattr(B, name)(a, b, *extra)

    def __add__(self, other):
        return self._binary("add", other, False, 1)

    def __radd__(self, other):
        return self._binary("add", other, True, 1)

    def __sub__(self, other):
        return self._binary("sub", other, False, 1)

    def __rsub__(self, other):
        return self._binary("sub", other, True, 1)

    def __mul__(self, other):
        return self._binary("mul", other)

    def __rmul__(self, other):
        return self._binary("mul", other, True)

    def __truediv__(self, other):
        return self._binary("div", other)

    def __rtruediv__(self, other):
        return self._binary("div", other, True)

    def __pow__(self, other):
        return self._binary("pow", other)

    def __rpow__(self, other):
        return self._binary("pow", other, True)

    def max(self, dim=None, keepdim=False):
        from mytorch_b200.ops.max import max as func

        return func(self, dim, keepdim)

    def eq(self, other):
        from mytorch_b200.ops.eq import eq as func

        return func(self, self._cast_other_to_tensor(other))

    def backward(self):
        DAGTracker.instance().backward(self)
