"""conv2d front-end (``mytorch/nn/functional/conv.py:10-49``)."""
from mytorch_b200.ops._common import dispatch, grad_enabled, record, tracker
from mytorch_b200.tensor import MismatchDataTypesError, MismatchDevicesError, Tensor


def conv2d(input: Tensor, weight: Tensor, bias=None, stride=1, padding=0, bn_stats=False) -> Tensor:
    """``bn_stats`` (no counterpart in the reference): the result goes straight into a BatchNorm layer
    in training mode; the CUDA backend then lets the convolution reduce the batch statistics of its
    own output, which BatchNorm picks up instead of re-reading the tensor.  Results are unchanged."""
    tensors = [input, weight] + ([bias] if bias is not None else [])
    if any(t.device != input.device for t in tensors):
        raise MismatchDevicesError([t.device for t in tensors])
    if any(t.dtype != input.dtype for t in tensors):
        raise MismatchDataTypesError([t.dtype for t in tensors])
    stride = (stride, stride) if isinstance(stride, int) else tuple(stride)
    padding = (padding, padding) if isinstance(padding, int) else tuple(padding)
    if bn_stats and input.device.type == "cuda":
        out = dispatch(input.device, "conv2d")(input, weight, bias, stride, padding, bn_stats=True)
    else:
        out = dispatch(input.device, "conv2d")(input, weight, bias, stride, padding)
    out.requires_grad = grad_enabled(input, weight, bias)
    return record("conv2d", [input, weight, bias, stride, padding], out)


@tracker.register_backward_function("conv2d")
def conv2d_backward(output_grad, input, weight, bias, stride, padding, accumulate_dx=None, defer_weight_gradient=False):
    """``accumulate_dx`` is the gradient ``input`` already holds (the tape passes it for operators
    listed in ``DAGTracker.fused_accumulate``): the returned dx then includes it.
    ``defer_weight_gradient`` (passed by the tape for operators in ``DAGTracker.deferrable``): the backend
    may compute dw beside the rest of the pass; it is complete after the tape's next ``join_hook()``."""
    backend = dispatch(input.device, "conv2d_backward")
    extra = {}
    if accumulate_dx is not None:
        extra["accumulate_dx"] = accumulate_dx
    if defer_weight_gradient and input.device.type == "cuda":
        extra["defer_weight_gradient"] = True
    dx, dw, db = backend(output_grad, input, weight, bias, stride, padding, **extra)
    return [dx, dw, db]


tracker.fused_accumulate["conv2d"] = 0  # input 0's accumulated gradient can be folded into the backward
tracker.deferrable.add("conv2d")        # the weight gradient may run beside the rest of backward
