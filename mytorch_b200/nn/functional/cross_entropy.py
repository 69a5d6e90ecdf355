"""Softmax cross-entropy front-end (``mytorch/nn/functional/cross_entropy.py:7-25``)."""
from mytorch_b200.dtype import int64
from mytorch_b200.ops._common import dispatch, grad_enabled, record, tracker
from mytorch_b200.tensor import InvalidDataTypeError, Tensor


def cross_entropy(input: Tensor, target: Tensor) -> Tensor:
    if target.dtype != int64:
        raise InvalidDataTypeError(target.dtype)
    out = dispatch(input.device, "cross_entropy")(input, target)
    out.requires_grad = grad_enabled(input)
    return record("cross_entropy", [input, target], out)


@tracker.register_backward_function("cross_entropy")
def cross_entropy_backward(output_grad, input, target):
    return dispatch(input.device, "cross_entropy_backward")(output_grad, input, target)
