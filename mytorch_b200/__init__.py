"""mytorch_b200 — the CNN training-step path of tigert1998/mytorch rebuilt for NVIDIA B200.

The Python surface is the reference's (``mytorch/__init__.py:1-23``): ``Tensor`` / ``tensor``,
``no_grad``, dtypes, ``mm`` / ``permute`` / ``reshape`` / ``add`` …, with ``mytorch_b200.nn``,
``mytorch_b200.nn.functional`` and ``mytorch_b200.optim`` beside it.  Every CUDA operator runs in
``lib/libmytorch_b200.so`` (hand-written sm_100a kernels behind a C ABI).
"""
from .autograd import no_grad
from .dtype import (DType, float16, float32, float64, int8, int16, int32, int64, uint8, uint16, uint32, uint64)
from .rand_generator import manual_seed
from .tensor import Device, Tensor, tensor
from .ops.basic_ops import bmm, mm, permute, reshape
from .ops.eq import eq
from .ops.max import max
from .ops.broadcast_binary_ops import add, div, mul, pow, sub
from .ops.reduce_ops import mean, sum
from .serialization import load, save

__all__ = ["Tensor", "tensor", "Device", "no_grad", "manual_seed", "mm", "bmm", "permute", "reshape", "max", "eq", "add", "sub", "mul", "div", "pow",
           "sum", "mean", "save", "load", "DType", "float16", "float32", "float64", "int8", "int16", "int32", "int64", "uint8",
           "uint16", "uint32", "uint64"]
