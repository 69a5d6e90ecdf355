"""dtype cast front-end (``mytorch/ops/cast.py:12-36``)."""
from mytorch_b200.dtype import DType
from mytorch_b200.ops._common import dispatch, record, tracker
from mytorch_b200.tensor import Tensor


def _cast(x: Tensor, dtype: DType):
    if x.dtype == dtype:
        return x
    out = dispatch(x.device, "cast")(x, dtype)
    out.requires_grad = x.requires_grad and x.dtype.is_floating and dtype.is_floating and not tracker.no_grad
    return record("cast", [x, dtype], out)


@tracker.register_backward_function("cast")
def _cast_backward(output_grad, x, dtype):
    return [dispatch(x.device, "cast")(output_grad, x.dtype)]
