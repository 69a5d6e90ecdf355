from mytorch_b200.ops._common import dispatch, grad_enabled, record, tracker
from mytorch_b200.ops.elementwise_ops import _relu
from mytorch_b200.tensor import MismatchDevicesError


def relu(x):
    return _relu(x)


def add_relu(x, y):
    """relu(x + y) for two tensors of the same shape, in one pass (residual connections)."""
    if x.device != y.device:
        raise MismatchDevicesError([x.device, y.device])
    out = dispatch(x.device, "add_relu")(x, y)
    out.requires_grad = grad_enabled(x, y)
    return record("add_relu", [x, y], out)


@tracker.register_backward_function("add_relu")
def add_relu_backward(output_grad, x, y):
    return dispatch(x.device, "add_relu_backward")(output_grad, x, y)
