"""Conv2d layer (``mytorch/nn/conv.py:11-72``): weight [Cout, Cin, KH, KW], optional bias,
Kaiming-uniform(a=sqrt 5) weight and U(-1/sqrt(fan_in), 1/sqrt(fan_in)) bias."""
import math

import numpy as np

import mytorch_b200 as mytorch
from mytorch_b200.nn.functional.conv import conv2d
from mytorch_b200.nn.init import _calculate_fan_in_and_fan_out, kaiming_uniform_
from mytorch_b200.nn.module import Module
from mytorch_b200.nn.parameter import Parameter


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class Conv2d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, bias=True, device="cpu", dtype=None):
        super().__init__()
        dtype = mytorch.float32 if dtype is None else dtype
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding = _pair(kernel_size), _pair(stride), _pair(padding)
        self.register_parameter("weight", Parameter(mytorch.tensor(
            np.zeros((out_channels, in_channels, *self.kernel_size)), dtype=dtype, device=device)))
        self.register_parameter("bias", Parameter(mytorch.tensor(np.zeros((out_channels,)), dtype=dtype, device=device)) if bias else None)
        # set by a model whose next layer is a BatchNorm: lets the CUDA convolution hand that layer its
        # batch statistics (see nn.functional.conv2d); purely an optimisation, results are unchanged
        self.feeds_batch_norm = False
        self.reset_parameters()

    def reset_parameters(self):
        kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in, _ = _calculate_fan_in_and_fan_out(self.weight)
            if fan_in != 0:
                bound = 1 / math.sqrt(fan_in)
                self.bias.uniform_(-bound, bound)

    def forward(self, input):
        return conv2d(input, self.weight, self.bias, self.stride, self.padding, bn_stats=self.feeds_batch_norm and self.training)
