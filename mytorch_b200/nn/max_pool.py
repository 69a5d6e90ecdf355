"""MaxPool2d (``mytorch/nn/max_pool.py:5-21``; note the default stride is 1, as there)."""
from mytorch_b200.nn.functional.pool_ops import max_pool2d
from mytorch_b200.nn.module import Module


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class MaxPool2d(Module):
    def __init__(self, kernel_size, stride=1, padding=0):
        super().__init__()
        self.kernel_size, self.stride, self.padding = _pair(kernel_size), _pair(stride), _pair(padding)

    def forward(self, input):
        return max_pool2d(input, kernel_size=self.kernel_size, stride=self.stride, padding=self.padding)
