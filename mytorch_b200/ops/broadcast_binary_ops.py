"""add / sub / mul / div / pow with NumPy broadcasting, and ``copy``
(signatures of ``mytorch/ops/broadcast_binary_ops.py:9-122``)."""
from mytorch_b200.ops._common import dispatch, grad_enabled, record, tracker
from mytorch_b200.tensor import MismatchDevicesError, Tensor


def _binary(name, x, y, *extra):
    if x.device != y.device:
        raise MismatchDevicesError([x.device, y.device])
    z = dispatch(x.device, name)(x, y, *extra)
    z.requires_grad = grad_enabled(x, y)
    return record(name, [x, y, *extra], z)


def add(x: Tensor, y: Tensor, alpha) -> Tensor:
    return _binary("add", x, y, alpha)


def sub(x: Tensor, y: Tensor, alpha) -> Tensor:
    return _binary("sub", x, y, alpha)


def mul(x: Tensor, y: Tensor) -> Tensor:
    return _binary("mul", x, y)


def div(x: Tensor, y: Tensor) -> Tensor:
    return _binary("div", x, y)


def pow(x: Tensor, y: Tensor) -> Tensor:
    return _binary("pow", x, y)


@tracker.register_backward_function("add")
def add_backward(output_grad, x, y, alpha):
    return dispatch(x.device, "add_backward")(output_grad, x, y, alpha)


@tracker.register_backward_function("sub")
def sub_backward(output_grad, x, y, alpha):
    return dispatch(x.device, "sub_backward")(output_grad, x, y, alpha)


@tracker.register_backward_function("mul")
def mul_backward(output_grad, x, y):
    return dispatch(x.device, "mul_backward")(output_grad, x, y)


@tracker.register_backward_function("div")
def div_backward(output_grad, x, y):
    return dispatch(x.device, "div_backward")(output_grad, x, y)


@tracker.register_backward_function("pow")
def pow_backward(output_grad, x, y):
    return dispatch(x.device, "pow_backward")(output_grad, x, y)


def _copy(x: Tensor, y: Tensor):
    if x.device != y.device:
        raise MismatchDevicesError([x.device, y.device])
    dispatch(x.device, "copy")(x, y)
