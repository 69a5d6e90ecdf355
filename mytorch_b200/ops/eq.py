"""eq front-end (``mytorch/ops/eq.py:5-11``): element-wise equality as an int8 tensor, no gradient."""
from mytorch_b200.ops._common import dispatch
from mytorch_b200.tensor import MismatchDataTypesError, Tensor


def eq(x: Tensor, y: Tensor):
    if x.dtype != y.dtype:
        raise MismatchDataTypesError([x.dtype, y.dtype])
    return dispatch(x.device, "eq")(x, y)
