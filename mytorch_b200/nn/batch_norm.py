"""BatchNorm2d (``mytorch/nn/batch_norm.py:7-135``): affine weight=1 / bias=0, running mean 0 /
running var 1; training mode normalises with batch statistics and blends the *biased* batch
variance into ``running_var``."""
from mytorch_b200.dtype import float32
from mytorch_b200.nn.functional.batch_norm import _batch_norm2d, _batch_norm2d_add_relu, _batch_norm2d_relu
from mytorch_b200.nn.module import Module
from mytorch_b200.nn.parameter import Parameter
from mytorch_b200.tensor import Tensor


class BatchNorm2d(Module):
    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, track_running_stats=True, device="cpu", dtype=float32):
        super().__init__()
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.affine, self.track_running_stats = affine, track_running_stats
        if affine:
            self.weight = Parameter(Tensor(shape=(num_features,), dtype=dtype, device=device))
            self.bias = Parameter(Tensor(shape=(num_features,), dtype=dtype, device=device))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        if track_running_stats:
            self.running_mean = Tensor(shape=(num_features,), dtype=dtype, device=device)
            self.running_var = Tensor(shape=(num_features,), dtype=dtype, device=device)
        else:
            self.register_buffer("running_mean", None)
            self.register_buffer("running_var", None)
        self.reset_parameters()

    def reset_parameters(self):
        if self.track_running_stats:
            self.running_mean.fill_(0)
            self.running_var.fill_(1)
        if self.affine:
            self.weight.fill_(1)
            self.bias.fill_(0)

    def forward(self, x):
        return _batch_norm2d(x, self.weight, self.bias, self.eps, self.training, self.momentum, self.running_mean, self.running_var)


class BatchNormReLU2d(BatchNorm2d):
    """``BatchNorm2d`` immediately followed by ``ReLU`` as one fused operator.  Same parameters,
    buffers and state-dict keys as ``BatchNorm2d``; results equal ``ReLU()(BatchNorm2d(...)(x))``."""

    def forward(self, x):
        return _batch_norm2d_relu(x, self.weight, self.bias, self.eps, self.training, self.momentum, self.running_mean, self.running_var)


class BatchNormAddReLU2d(BatchNorm2d):
    """The tail of a residual block as one fused operator: ``forward(x, residual)`` returns
    ``ReLU()(BatchNorm2d(...)(x) + residual)``.  Same parameters, buffers and state-dict keys as ``BatchNorm2d``."""

    def forward(self, x, residual):
        return _batch_norm2d_add_relu(x, residual, self.weight, self.bias, self.eps, self.training, self.momentum, self.running_mean,
                                      self.running_var)


class BatchNorm1d(BatchNorm2d):
    """BatchNorm over [N, C] or [N, C, L] inputs (``mytorch/nn/batch_norm.py:92-106``): the same per-channel
    statistics over every non-channel dimension, computed by the BatchNorm2d kernels on the input viewed
    as [N, C, L, 1]."""

    def forward(self, x):
        if len(x.shape) not in (2, 3):
            raise RuntimeError(f"BatchNorm1d expects a 2-D or 3-D input, got shape {x.shape}")
        n, c = x.shape[0], x.shape[1]
        length = x.shape[2] if len(x.shape) == 3 else 1
        y = _batch_norm2d(x.reshape((n, c, length, 1)), self.weight, self.bias, self.eps, self.training, self.momentum, self.running_mean,
                          self.running_var)
        return y.reshape(x.shape)
