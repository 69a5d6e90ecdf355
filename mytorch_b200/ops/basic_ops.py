"""mm / bmm / permute / reshape front-ends (signatures of ``mytorch/ops/basic_ops.py:12-106``)."""
from mytorch_b200.ops._common import dispatch, grad_enabled, record, tracker
from mytorch_b200.tensor import MismatchDevicesError, Tensor


def mm(x: Tensor, y: Tensor) -> Tensor:
    if x.device != y.device:
        raise MismatchDevicesError([x.device, y.device])
    z = dispatch(x.device, "mm")(x, y)
    z.requires_grad = grad_enabled(x, y)
    return record("mm", [x, y], z)


@tracker.register_backward_function("mm")
def mm_backward(output_grad, x, y):
    if not (output_grad.device == x.device == y.device):
        raise MismatchDevicesError([output_grad.device, x.device, y.device])
    x_grad, y_grad = dispatch(x.device, "mm_backward")(output_grad, x, y)
    return [x_grad, y_grad]


def bmm(x: Tensor, y: Tensor) -> Tensor:
    """Batched matrix product [B,M,K] x [B,K,N] (``mytorch/ops/basic_ops.py:39-63``)."""
    if x.device != y.device:
        raise MismatchDevicesError([x.device, y.device])
    z = dispatch(x.device, "bmm")(x, y)
    z.requires_grad = grad_enabled(x, y)
    return record("bmm", [x, y], z)


@tracker.register_backward_function("bmm")
def bmm_backward(output_grad, x, y):
    if not (output_grad.device == x.device == y.device):
        raise MismatchDevicesError([output_grad.device, x.device, y.device])
    x_grad, y_grad = dispatch(x.device, "bmm_backward")(output_grad, x, y)
    return [x_grad, y_grad]


def permute(x: Tensor, dims) -> Tensor:
    if len(dims) != len(x.shape):
        raise RuntimeError(f"permute dims is invalid: {dims}")
    dims = tuple(d + len(dims) if d < 0 else d for d in dims)
    out = dispatch(x.device, "permute")(x, dims)
    out.requires_grad = grad_enabled(x)
    return record("permute", [x, dims], out)


@tracker.register_backward_function("permute")
def permute_backward(output_grad, x, dims):
    (g,) = dispatch(x.device, "permute_backward")(output_grad, x, dims)
    return [g]


def reshape(x: Tensor, shape) -> Tensor:
    out = dispatch(x.device, "reshape")(x, shape)
    out.requires_grad = grad_enabled(x)
    return record("reshape", [x, out.shape], out)


@tracker.register_backward_function("reshape")
def reshape_backward(output_grad, x, shape):
    return [dispatch(x.device, "reshape")(output_grad, x.shape)]
