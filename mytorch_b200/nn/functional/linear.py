"""y = x Wᵀ + b as one operator.

The reference's ``nn.Linear`` composes reshape, permute (a kernel that copies Wᵀ every step),
mm and a broadcast add (``mytorch/nn/linear.py:59-65``).  Here the GEMM reads W as stored
(K-major) and adds the bias in its epilogue; backward produces dX, dW and db directly.
"""
from mytorch_b200.ops._common import dispatch, grad_enabled, record, tracker
from mytorch_b200.tensor import MismatchDevicesError, Tensor


def linear(x: Tensor, weight: Tensor, bias=None) -> Tensor:
    if x.device != weight.device or (bias is not None and bias.device != x.device):
        raise MismatchDevicesError([x.device, weight.device])
    out = dispatch(x.device, "linear")(x, weight, bias)
    out.requires_grad = grad_enabled(x, weight, bias)
    return record("linear", [x, weight, bias], out)


@tracker.register_backward_function("linear")
def linear_backward(output_grad, x, weight, bias):
    return dispatch(x.device, "linear_backward")(output_grad, x, weight, bias)
