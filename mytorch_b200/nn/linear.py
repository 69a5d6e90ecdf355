"""Linear layer (``mytorch/nn/linear.py:12-65``): weight [out, in], same initialisation; the
forward is one fused GEMM+bias operator instead of reshape/permute/mm/add."""
import math

import numpy as np

import mytorch_b200 as mytorch
from mytorch_b200.nn.functional.linear import linear
from mytorch_b200.nn.init import _calculate_fan_in_and_fan_out, kaiming_uniform_
from mytorch_b200.nn.module import Module
from mytorch_b200.nn.parameter import Parameter
from mytorch_b200.ops.basic_ops import reshape


class Linear(Module):
    def __init__(self, in_features, out_features, bias=True, device="cpu", dtype=None):
        super().__init__()
        dtype = mytorch.float32 if dtype is None else dtype
        self.in_features, self.out_features = in_features, out_features
        self.register_parameter("weight", Parameter(mytorch.tensor(np.zeros((out_features, in_features)), dtype=dtype, device=device)))
        self.register_parameter("bias", Parameter(mytorch.tensor(np.zeros((out_features,)), dtype=dtype, device=device)) if bias else None)
        self.reset_parameters()

    def reset_parameters(self):
        kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in, _ = _calculate_fan_in_and_fan_out(self.weight)
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            self.bias.uniform_(-bound, bound)

    def forward(self, x):
        lead = x.shape[:-1]
        if len(x.shape) != 2:
            x = reshape(x, (-1, self.in_features))
        y = linear(x, self.weight, self.bias)
        if len(lead) != 1:
            y = reshape(y, lead + (self.out_features,))
        return y
