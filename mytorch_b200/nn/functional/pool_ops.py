"""max_pool2d front-end (``mytorch/nn/functional/pool_ops.py:5-21``): the output is kept as the
backward's helper tensor, as in the reference."""
from mytorch_b200.ops._common import dispatch, grad_enabled, record, tracker


def max_pool2d(x, kernel_size, stride=None, padding=0):
    out = dispatch(x.device, "max_pool2d")(x, kernel_size, stride, padding)
    out.requires_grad = grad_enabled(x)
    return record("max_pool2d", [x, kernel_size, stride, padding], out, [out])


@tracker.register_backward_function("max_pool2d")
def max_pool2d_backward(output_grad, output, input, kernel_size, stride, padding):
    return dispatch(input.device, "max_pool2d_backward")(output_grad, output, input, kernel_size, stride, padding)
