"""max front-end (``mytorch/ops/max.py:5-26``): ``max(t, dim)`` returns (values, int64 indices along
``dim``); ``max(t)`` returns the largest element.  Backward sends the gradient to the recorded index."""
from mytorch_b200.ops._common import dispatch, grad_enabled, tracker


def max(tensor, dim=None, keepdim=False):
    output, indices = dispatch(tensor.device, "max")(tensor, dim, keepdim)
    output.requires_grad = grad_enabled(tensor)
    if output.requires_grad:
        tracker.add_node("max", [tensor, dim, keepdim], [output], [indices])
    return (output, indices) if dim is not None else output


@tracker.register_backward_function("max")
def max_backward(output_grad, indices_tensor, tensor, dim, keepdim):
    return dispatch(tensor.device, "max_backward")(output_grad, indices_tensor, tensor, dim, keepdim)
