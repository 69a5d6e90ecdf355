"""sum / mean through ``sum_scale`` (signatures of ``mytorch/ops/reduce_ops.py:9-42``)."""
from mytorch_b200.ops._common import dispatch, grad_enabled, record, tracker
from mytorch_b200.tensor import Tensor, shape_size


def _dims(x, dim):
    if dim is None:
        return tuple(range(len(x.shape)))
    return (dim,) if isinstance(dim, int) else tuple(dim)


def _sum_scale(x: Tensor, dim=None, keepdim=False, scale=1) -> Tensor:
    dim = _dims(x, dim)
    out = dispatch(x.device, "sum_scale")(x, dim, keepdim, scale)
    out.requires_grad = grad_enabled(x)
    return record("sum_scale", [x, dim, keepdim, scale], out)


@tracker.register_backward_function("sum_scale")
def _sum_scale_backward(output_grad, x, dim=None, keepdim=False, scale=1):
    return dispatch(x.device, "sum_scale_backward")(output_grad, x, dim, keepdim, scale)


def sum(x: Tensor, dim=None, keepdim=False) -> Tensor:
    return _sum_scale(x, dim, keepdim, 1)


def mean(x: Tensor, dim=None, keepdim=False) -> Tensor:
    dim = _dims(x, dim)
    return _sum_scale(x, dim, keepdim, 1 / shape_size([x.shape[i] for i in dim]))
