"""Fused BatchNorm2d front-end (``mytorch/nn/functional/batch_norm.py:8-51``)."""
from mytorch_b200.ops._common import dispatch, record, tracker
from mytorch_b200.tensor import Tensor


def _batch_norm2d(input: Tensor, weight, bias, eps, training, momentum, running_mean, running_var):
    requires_grad = input.requires_grad
    channels = input.shape[1]
    if weight is not None and bias is not None:
        ok = (input.dtype == weight.dtype == bias.dtype and input.device == weight.device == bias.device
              and weight.shape == (channels,) and bias.shape == (channels,))
        if not ok:
            raise RuntimeError("batch_norm2d shape, dtype or device mismatch")
        requires_grad = requires_grad or weight.requires_grad or bias.requires_grad
    out, mean, var = dispatch(input.device, "batch_norm2d")(input, weight, bias, eps, training, momentum, running_mean, running_var)
    out.requires_grad = requires_grad and not tracker.no_grad
    return record("batch_norm2d", [input, weight, bias, eps], out, [mean, var])


@tracker.register_backward_function("batch_norm2d")
def _batch_norm2d_backward(output_grad, mean, var, input, weight, bias, eps):
    return dispatch(input.device, "batch_norm2d_backward")(output_grad, mean, var, input, weight, bias, eps)


def _batch_norm2d_relu(input: Tensor, weight, bias, eps, training, momentum, running_mean, running_var):
    """relu(batch_norm2d(x)) as one operator: the normalise pass applies max(0, .) before it stores,
    and backward re-derives the ReLU mask from x, so the intermediate is never written or read.
    Same arithmetic as ``BatchNorm2d`` followed by ``ReLU`` (``mytorch/nn/batch_norm.py:123-135``,
    ``mytorch/nn/relu.py:5-10``); the reference runs them as two operators."""
    requires_grad = input.requires_grad
    channels = input.shape[1]
    if weight is not None and bias is not None:
        ok = (input.dtype == weight.dtype == bias.dtype and input.device == weight.device == bias.device
              and weight.shape == (channels,) and bias.shape == (channels,))
        if not ok:
            raise RuntimeError("batch_norm2d shape, dtype or device mismatch")
        requires_grad = requires_grad or weight.requires_grad or bias.requires_grad
    out, mean, var = dispatch(input.device, "batch_norm2d_relu")(input, weight, bias, eps, training, momentum, running_mean, running_var)
    out.requires_grad = requires_grad and not tracker.no_grad
    return record("batch_norm2d_relu", [input, weight, bias, eps], out, [mean, var])


@tracker.register_backward_function("batch_norm2d_relu")
def _batch_norm2d_relu_backward(output_grad, mean, var, input, weight, bias, eps):
    return dispatch(input.device, "batch_norm2d_relu_backward")(output_grad, mean, var, input, weight, bias, eps)


def _batch_norm2d_add_relu(input: Tensor, residual: Tensor, weight, bias, eps, training, momentum, running_mean, running_var):
    """relu(batch_norm2d(x) + residual) as one operator: the tail of a residual block.  The reference runs
    three operators (``mytorch/nn/batch_norm.py:123-135``, ``mytorch/tensor.py:292-300``,
    ``mytorch/nn/relu.py:5-10``); here the BatchNorm output and the sum are never stored, and backward
    re-derives the ReLU mask from x, the statistics and the residual."""
    channels = input.shape[1]
    requires_grad = input.requires_grad or residual.requires_grad
    if input.shape != residual.shape or input.device != residual.device or input.dtype != residual.dtype:
        raise RuntimeError("batch_norm2d_add_relu: x and the tensor to add must agree in shape, dtype and device")
    if weight is not None and bias is not None:
        ok = (input.dtype == weight.dtype == bias.dtype and input.device == weight.device == bias.device
              and weight.shape == (channels,) and bias.shape == (channels,))
        if not ok:
            raise RuntimeError("batch_norm2d shape, dtype or device mismatch")
        requires_grad = requires_grad or weight.requires_grad or bias.requires_grad
    out, mean, var = dispatch(input.device, "batch_norm2d_add_relu")(input, residual, weight, bias, eps, training, momentum, running_mean, running_var)
    out.requires_grad = requires_grad and not tracker.no_grad
    return record("batch_norm2d_add_relu", [input, residual, weight, bias, eps], out, [mean, var])


@tracker.register_backward_function("batch_norm2d_add_relu")
def _batch_norm2d_add_relu_backward(output_grad, mean, var, input, residual, weight, bias, eps):
    return dispatch(input.device, "batch_norm2d_add_relu_backward")(output_grad, mean, var, input, residual, weight, bias, eps)
