"""fill / normal / uniform / relu front-ends (``mytorch/ops/elementwise_ops.py:9-38``)."""
from mytorch_b200.ops._common import dispatch, grad_enabled, record, tracker
from mytorch_b200.tensor import Tensor


def _fill(x: Tensor, value):
    dispatch(x.device, "fill")(x, value)


def _normal(x: Tensor, seed, mean, stddev):
    dispatch(x.device, "normal")(x, seed, mean, stddev)


def _uniform(x: Tensor, seed, a, b):
    dispatch(x.device, "uniform")(x, seed, a, b)


def _relu(x: Tensor) -> Tensor:
    out = dispatch(x.device, "relu")(x)
    out.requires_grad = grad_enabled(x)
    return record("relu", [x], out)


@tracker.register_backward_function("relu")
def relu_backward(output_grad, x):
    return dispatch(output_grad.device, "relu_backward")(output_grad, x)
