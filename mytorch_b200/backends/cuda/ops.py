"""CUDA operator wrappers: allocate outputs, marshal shapes and scalars, call the kernel library.

One function per registry name, with the positional signatures and return containers of the
reference's ``mytorch/backends/cuda/ops/*.py`` (e.g. ``conv2d`` / ``conv2d_backward``
``conv.py:9-90``, ``batch_norm2d`` ``batch_norm.py:10-105``, ``max_pool2d`` ``pool_ops.py:95-104``,
``sgd`` ``sgd.py:8-35``).  No wrapper synchronises, copies metadata to the device or touches the
host copy of a tensor, so a whole training step can be captured in a CUDA graph.

4-D float32 tensors are channels-last in device memory (see ``tensor.py``); helpers below give
the logical-dimension strides of either layout to the generic strided kernels.
"""
from __future__ import annotations

import ctypes

import numpy as np

from mytorch_b200.backends.backend_dispatcher import BackendDispatcher
from mytorch_b200.backends.cuda.env import CudaEnv, CudaMemory
from mytorch_b200.backends.utils import calculate_broadcast_shape, calculate_reduce_shape, calculate_reshaped_shape
from mytorch_b200.dtype import float32, int32, int64

_reg = BackendDispatcher.instance().register_backend_function
_LL = ctypes.c_longlong


def _T():
    from mytorch_b200.tensor import Tensor

    return Tensor


def _env(t=None):
    env = CudaEnv.instance()
    if t is not None:
        env.set_device(t.device.index)
    return env


def _ptr(t):
    return None if t is None else t._native_array.ptr


def _numel(shape):
    n = 1
    for s in shape:
        n *= s
    return n


def _new(shape, like, dtype=None):
    return _T()(shape=tuple(shape), dtype=dtype or like.dtype, device=like.device)


def _grad_buffer(param):
    """Output tensor for a parameter's gradient.  Under the data-parallel wrapper every parameter
    owns a window of the flat all-reduce buffer (``param._grad_slot``) and its first gradient of a
    backward pass is written straight into it; otherwise (no wrapper, or a second contribution that
    the tape will add to the first) a fresh tensor."""
    slot = getattr(param, "_grad_slot", None)
    if slot is None or param.grad is not None:
        return _new(param.shape, param)
    g = _T()(tensor=param)
    g._native_array = slot
    return g


def _f32(*tensors):
    from mytorch_b200.tensor import InvalidDataTypeError

    for t in tensors:
        if t is not None and t.dtype is not float32:
            raise InvalidDataTypeError(t.dtype)


def _nontrivial_nhwc(t):
    return t._nhwc and t.shape[1] > 1 and t.shape[2] * t.shape[3] > 1


def _strides(t):
    """Element strides of the logical dimensions in device memory."""
    shape = t.shape
    if t._nhwc:
        n, c, h, w = shape
        return [h * w * c, 1, w * c, c]
    out, acc = [0] * len(shape), 1
    for i in range(len(shape) - 1, -1, -1):
        out[i] = acc
        acc *= shape[i]
    return out


def _ll(values):
    return (_LL * max(len(values), 1))(*values)


# ---------------------------------------------------------------------------- host <-> device

@_reg("cuda", "upload")
def cuda_upload(t, array):
    """Host ndarray (logical layout) -> device storage of ``t`` (channels-last when 4-D float32)."""
    env = _env(t)
    array = np.ascontiguousarray(array, dtype=t.dtype.np_dtype)
    if _nontrivial_nhwc(t):
        stage = CudaMemory(t.device.index, array.nbytes)
        stage.write(array)
        n, c, h, w = t.shape
        env.lib.nchw_to_nhwc_f32(stage.ptr, _ptr(t), n, c, h, w, env.stream())
    else:
        t._native_array.write(array)


def upload_into(t, host):
    """Asynchronously refill an existing device tensor from host memory holding the logical (NCHW)
    layout: a NumPy array (page-locked, e.g. ``env.PinnedBuffer(...).array``, for a truly asynchronous
    copy) or an object with ``data_ptr()`` such as a pinned PyTorch CPU tensor.  The memory must stay
    valid until the copy has run.  The staging buffer of a channels-last tensor is allocated once and reused."""
    env = _env(t)
    src = host if hasattr(host, "data_ptr") else np.ascontiguousarray(host)
    if _nontrivial_nhwc(t):
        stage = getattr(t, "_stage", None)
        if stage is None:
            stage = t._stage = CudaMemory(t.device.index, t._native_array.nbytes)
        stage.write_from(src)
        n, c, h, w = t.shape
        env.lib.nchw_to_nhwc_f32(stage.ptr, _ptr(t), n, c, h, w, env.stream())
    else:
        t._native_array.write_from(src)
        if not hasattr(host, "data_ptr") and src is not host:
            env.lib.stream_synchronize(env.stream())  # `src` is a temporary: let the copy finish before it goes away


@_reg("cuda", "download")
def cuda_download(t):
    env = _env(t)
    if _nontrivial_nhwc(t):
        tmp = CudaMemory(t.device.index, t._native_array.nbytes)
        n, c, h, w = t.shape
        env.lib.nhwc_to_nchw_f32(_ptr(t), tmp.ptr, n, c, h, w, env.stream())
        return tmp.read(t.shape, t.dtype.np_dtype)
    return t._native_array.read(t.shape, t.dtype.np_dtype)


# ---------------------------------------------------------------------------- convolution

def _conv_args(x, w, stride, padding, cin=None):
    """(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout); `cin` overrides the filter's channel count when
    the activation has been padded to a channel block but the filter has not."""
    n, cin_x, h, wd = x.shape
    cout, cin2, kh, kw = w.shape
    if cin is not None:
        cin2 = cin
    cin = cin_x
    if cin != cin2:
        from mytorch_b200.tensor import MismatchShapesError

        raise MismatchShapesError([x.shape, w.shape])
    return (n, cin, h, wd, kh, kw, stride[0], stride[1], padding[0], padding[1], cout)


_TC_CHANNELS = 32  # the tensor-core convolution reads activations in blocks of 32 channels


def _wants_channel_padding(x):
    """Image stems (1 or 3 input channels) would otherwise run on the CUDA-core kernels; padding
    their few channels with zeros up to one 32-channel block lets them use the tensor-core path
    (extra zero FLOPs are far cheaper than the FFMA kernel) when the padded tensor is large enough
    for that path to accept it."""
    n, c, h, w = x.shape
    return c < _TC_CHANNELS and n * h * w * _TC_CHANNELS * 4 >= (1 << 17)


def _pad_channels(env, t, channels):
    """A channels-last tensor copied into one with `channels` channels (dim 1), the new ones zero."""
    n, c, h, w = t.shape
    out = _new((n, channels, h, w), t)
    env.lib.resize_channels_f32(_ptr(t), _ptr(out), n * h * w, c, channels, env.stream())
    return out


def _take_channels(env, t, channels, like, out=None):
    """First `channels` channels (dim 1) of a channels-last tensor, as a new tensor (or into `out`)."""
    n, c, h, w = t.shape
    out = _new((n, channels, h, w), like) if out is None else out
    env.lib.resize_channels_f32(_ptr(t), _ptr(out), n * h * w, c, channels, env.stream())
    return out


@_reg("cuda", "conv2d")
def cuda_conv2d(input, weight, bias, stride, padding, bn_stats=False):
    """``bn_stats``: the output feeds a BatchNorm layer in training mode; where the kernel allows, the
    convolution's epilogue also reduces the per-channel batch statistics of the output and leaves them
    on the result (``_bn_partials``) for ``batch_norm2d``, which then skips its own pass over the tensor."""
    _f32(input, weight, bias)
    env = _env(input)
    x, wt = input, weight
    if _wants_channel_padding(input):
        x, wt = _pad_channels(env, input, _TC_CHANNELS), _pad_channels(env, weight, _TC_CHANNELS)
        input._padded_for_conv = x  # backward of this convolution reuses it (the weight gradient reads x again)
    a = _conv_args(x, wt, stride, padding)
    n, cin, h, w, kh, kw, sh, sw, ph, pw, cout = a
    oh, ow = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    out = _new((n, cout, oh, ow), input)
    ws, ws_bytes = env.workspace(env.lib.conv2d_workspace_bytes(*a))
    if bn_stats:
        partials = CudaMemory(input.device.index, env.lib.conv2d_stats_max_rows() * 3 * cout * 4)
        rows = ctypes.c_int(0)
        env.lib.conv2d_forward_stats_f32(*a, _ptr(x), _ptr(wt), _ptr(bias), _ptr(out), 0, partials.ptr, ctypes.byref(rows), ws, ws_bytes,
                                         env.stream())
        if rows.value > 0:
            out._bn_partials = (partials, rows.value)
        return out
    env.lib.conv2d_forward_f32(*a, _ptr(x), _ptr(wt), _ptr(bias), _ptr(out), 0, ws, ws_bytes, env.stream())
    return out


@_reg("cuda", "conv2d_backward")
def cuda_conv2d_backward(output_grad, input, weight, bias, stride, padding, accumulate_dx=None, defer_weight_gradient=False):
    """``accumulate_dx``: a gradient the input has already received from another consumer; when given,
    the returned dx is the data gradient PLUS that tensor (added in the convolution's epilogue where
    the kernel allows), and the caller stores it instead of adding the two itself.
    ``defer_weight_gradient``: the caller (the tape) does not need dw until it calls ``CudaEnv.join_side``;
    the weight gradient then runs on the device's side stream, beside whatever the caller enqueues next."""
    _f32(output_grad, input, weight)
    env = _env(input)
    want_dx, want_dw, cin = input.requires_grad, weight.requires_grad, input.shape[1]
    padded = _wants_channel_padding(input)
    x, wt = input, weight
    if padded:
        x = getattr(input, "_padded_for_conv", None)
        if x is None:
            x = _pad_channels(env, input, _TC_CHANNELS)
        else:
            del input._padded_for_conv
        if want_dx:  # the data gradient reads the (padded) filter; the weight gradient only needs its shape
            wt = _pad_channels(env, weight, _TC_CHANNELS)
    a = _conv_args(x, weight, stride, padding, cin=x.shape[1])
    st = env.stream()
    ws, ws_bytes = env.workspace(env.lib.conv2d_workspace_bytes(*a))
    dx = dw = db = None
    if want_dx:
        if accumulate_dx is not None and not padded and env.lib.conv2d_dgrad_accumulates_in_place(
                *a, _ptr(output_grad), _ptr(wt), _ptr(accumulate_dx)):
            # a filter smaller than its stride (the 1x1 / stride-2 shortcut) reaches only some pixels: it adds
            # to those in the gradient the input already holds, which is then the returned tensor
            dx = accumulate_dx
            env.lib.conv2d_dgrad_add_f32(*a, _ptr(output_grad), _ptr(wt), _ptr(dx), _ptr(dx), ws, ws_bytes, st)
        elif accumulate_dx is not None and not padded:
            dx = _new(x.shape, x)
            env.lib.conv2d_dgrad_add_f32(*a, _ptr(output_grad), _ptr(wt), _ptr(accumulate_dx), _ptr(dx), ws, ws_bytes, st)
        else:
            dx = _new(x.shape, x)
            env.lib.conv2d_dgrad_f32(*a, _ptr(output_grad), _ptr(wt), _ptr(dx), ws, ws_bytes, st)
            if padded:
                dx = _take_channels(env, dx, cin, dx)
            if accumulate_dx is not None:
                dx = BackendDispatcher.instance().dispatch("cuda", "add")(dx, accumulate_dx, 1)
    if want_dw:
        # Nothing in the rest of backward reads this layer's weight gradient, so it runs on the side
        # stream, beside the data-gradient / BatchNorm chain that the next layer waits for, and is
        # joined when backward ends (or before anything touches the gradient: see DAGTracker.backward).
        # A weight that already holds a gradient (shared weights) accumulates on the compute stream.
        wst, wws, wws_bytes = st, ws, ws_bytes
        if defer_weight_gradient and env.overlap_weight_gradients and weight.grad is None:
            wst = env.fork_side((x, output_grad))
            wws, wws_bytes = env.side_workspace(env.lib.conv2d_workspace_bytes(*a))
        if padded:
            wide = _new((weight.shape[0], _TC_CHANNELS) + tuple(weight.shape[2:]), weight)
            env.lib.conv2d_wgrad_f32(*a, _ptr(x), _ptr(output_grad), _ptr(wide), wws, wws_bytes, wst)
            dw = _grad_buffer(weight)
            env.lib.resize_channels_f32(_ptr(wide), _ptr(dw), weight.shape[0] * weight.shape[2] * weight.shape[3], _TC_CHANNELS, cin, wst)
            if wst is not st:
                env._side_keepalive.append(wide)
        else:
            dw = _grad_buffer(weight)
            env.lib.conv2d_wgrad_f32(*a, _ptr(x), _ptr(output_grad), _ptr(dw), wws, wws_bytes, wst)
    if bias is not None and bias.requires_grad:
        db = _colsum(env, output_grad, _numel(output_grad.shape) // a[-1], a[-1], bias, out=_grad_buffer(bias))
    return [dx, dw, db]


def _colsum(env, mat, rows, cols, like, scale=1.0, out=None):
    out = _new((cols,), like) if out is None else out
    ws, ws_bytes = env.workspace(env.lib.colsum_workspace_bytes(cols))
    env.lib.colsum_f32(_ptr(mat), rows, cols, scale, _ptr(out), ws, ws_bytes, env.stream())
    return out


# ---------------------------------------------------------------------------- linear / mm

def _gemm(env, m, n, k, a, ta, b, tb, bias, relu, c):
    env.lib.gemm_f32(m, n, k, _ptr(a), ta, _ptr(b), tb, _ptr(bias), relu, _ptr(c), env.stream())


@_reg("cuda", "linear")
def cuda_linear(x, weight, bias):
    _f32(x, weight, bias)
    env = _env(x)
    b, fin = x.shape
    fout = weight.shape[0]
    if weight.shape[1] != fin:
        from mytorch_b200.tensor import MismatchShapesError

        raise MismatchShapesError([x.shape, weight.shape])
    y = _new((b, fout), x)
    _gemm(env, b, fout, fin, x, 0, weight, 1, bias, 0, y)
    return y


@_reg("cuda", "linear_backward")
def cuda_linear_backward(output_grad, x, weight, bias):
    env = _env(x)
    b, fin = x.shape
    fout = weight.shape[0]
    dx = dw = db = None
    if x.requires_grad:
        dx = _new(x.shape, x)
        _gemm(env, b, fin, fout, output_grad, 0, weight, 0, None, 0, dx)
    if weight.requires_grad:
        dw = _grad_buffer(weight)
        _gemm(env, fout, fin, b, output_grad, 1, x, 0, None, 0, dw)
    if bias is not None and bias.requires_grad:
        db = _colsum(env, output_grad, b, fout, bias, out=_grad_buffer(bias))
    return [dx, dw, db]


@_reg("cuda", "mm")
def cuda_mm(x, y):
    _f32(x, y)
    env = _env(x)
    (m, k), (k2, n) = x.shape, y.shape
    if k != k2:
        from mytorch_b200.tensor import MismatchShapesError

        raise MismatchShapesError([x.shape, y.shape])
    z = _new((m, n), x)
    _gemm(env, m, n, k, x, 0, y, 0, None, 0, z)
    return z


@_reg("cuda", "mm_backward")
def cuda_mm_backward(output_grad, x, y):
    env = _env(x)
    (m, k), n = x.shape, y.shape[1]
    dx, dy = _new(x.shape, x), _new(y.shape, y)
    _gemm(env, m, k, n, output_grad, 0, y, 1, None, 0, dx)
    _gemm(env, k, n, m, x, 1, output_grad, 0, None, 0, dy)
    return dx, dy


# ---------------------------------------------------------------------------- batch norm

@_reg("cuda", "batch_norm2d")
def cuda_batch_norm2d(x, weight, bias, eps, training, momentum, running_mean, running_var, relu=False):
    _f32(x, weight, bias, running_mean, running_var)
    env = _env(x)
    n, c, h, w = x.shape
    y, mean, var = _new(x.shape, x), _new((c,), x), _new((c,), x)
    ws, ws_bytes = env.workspace(env.lib.batch_norm2d_workspace_bytes(n, c, h, w))
    # without running statistics the reference normalises with batch statistics in eval mode too
    # (``mytorch/backends/cpu/ops/batch_norm.py:40-46``)
    use_batch_stats = bool(training) or running_mean is None or running_var is None
    pre = getattr(x, "_bn_partials", None)
    if use_batch_stats and pre is not None:  # the convolution that produced x already reduced its statistics
        env.lib.batch_norm2d_forward_prestats_f32(n, c, h, w, _ptr(x), _ptr(weight), _ptr(bias), float(eps), float(momentum), _ptr(running_mean),
                                                  _ptr(running_var), _ptr(y), _ptr(mean), _ptr(var), int(bool(relu)), pre[0].ptr, pre[1], ws, ws_bytes,
                                                  env.stream())
        return y, mean, var
    env.lib.batch_norm2d_forward_f32(n, c, h, w, _ptr(x), _ptr(weight), _ptr(bias), float(eps), int(use_batch_stats), float(momentum),
                                     _ptr(running_mean), _ptr(running_var), _ptr(y), _ptr(mean), _ptr(var), int(bool(relu)), ws, ws_bytes, env.stream())
    return y, mean, var


@_reg("cuda", "batch_norm2d_add_relu")
def cuda_batch_norm2d_add_relu(x, residual, weight, bias, eps, training, momentum, running_mean, running_var):
    """max(0, batch_norm2d(x) + residual) in one normalise pass; returns (y, mean, var)."""
    _f32(x, residual, weight, bias, running_mean, running_var)
    if x.shape != residual.shape:
        from mytorch_b200.tensor import MismatchShapesError

        raise MismatchShapesError([x.shape, residual.shape])
    env = _env(x)
    n, c, h, w = x.shape
    y, mean, var = _new(x.shape, x), _new((c,), x), _new((c,), x)
    ws, ws_bytes = env.workspace(env.lib.batch_norm2d_workspace_bytes(n, c, h, w))
    use_batch_stats = bool(training) or running_mean is None or running_var is None
    pre = getattr(x, "_bn_partials", None) if use_batch_stats else None
    env.lib.batch_norm2d_add_relu_forward_f32(n, c, h, w, _ptr(x), _ptr(residual), _ptr(weight), _ptr(bias), float(eps), int(use_batch_stats),
                                              float(momentum), _ptr(running_mean), _ptr(running_var), _ptr(y), _ptr(mean), _ptr(var),
                                              pre[0].ptr if pre else None, pre[1] if pre else 0, ws, ws_bytes, env.stream())
    return y, mean, var


@_reg("cuda", "batch_norm2d_add_relu_backward")
def cuda_batch_norm2d_add_relu_backward(output_grad, mean, var, x, residual, weight, bias, eps):
    """[dx, dresidual, dgamma, dbeta]"""
    env = _env(x)
    n, c, h, w = x.shape
    dx, dres = _new(x.shape, x), _new(x.shape, x)
    affine = weight is not None and bias is not None
    dg = _grad_buffer(weight) if affine else None
    db = _grad_buffer(bias) if affine else None
    ws, ws_bytes = env.workspace(env.lib.batch_norm2d_workspace_bytes(n, c, h, w))
    env.lib.batch_norm2d_add_relu_backward_f32(n, c, h, w, _ptr(output_grad), _ptr(mean), _ptr(var), _ptr(x), _ptr(residual), _ptr(weight), _ptr(bias),
                                               float(eps), _ptr(dx), _ptr(dres), _ptr(dg), _ptr(db), ws, ws_bytes, env.stream())
    return [dx, dres, dg, db]


@_reg("cuda", "batch_norm2d_relu")
def cuda_batch_norm2d_relu(x, weight, bias, eps, training, momentum, running_mean, running_var):
    """BatchNorm2d followed by ReLU in one normalise pass (the ReLU input is never stored)."""
    return cuda_batch_norm2d(x, weight, bias, eps, training, momentum, running_mean, running_var, relu=True)


@_reg("cuda", "batch_norm2d_relu_backward")
def cuda_batch_norm2d_relu_backward(output_grad, mean, var, x, weight, bias, eps):
    return cuda_batch_norm2d_backward(output_grad, mean, var, x, weight, bias, eps, relu=True)


@_reg("cuda", "batch_norm2d_backward")
def cuda_batch_norm2d_backward(output_grad, mean, var, x, weight, bias, eps, relu=False):
    env = _env(x)
    n, c, h, w = x.shape
    dx = _new(x.shape, x)
    affine = weight is not None and bias is not None
    dg = _grad_buffer(weight) if affine else None
    db = _grad_buffer(bias) if affine else None
    ws, ws_bytes = env.workspace(env.lib.batch_norm2d_workspace_bytes(n, c, h, w))
    env.lib.batch_norm2d_backward_f32(n, c, h, w, _ptr(output_grad), _ptr(mean), _ptr(var), _ptr(x), _ptr(weight), _ptr(bias), float(eps),
                                      int(bool(relu)), _ptr(dx), _ptr(dg), _ptr(db), ws, ws_bytes, env.stream())
    return [dx, dg, db]


# ---------------------------------------------------------------------------- pooling

def _pool_args(x, kernel_size, stride, padding):
    pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)
    kh, kw = pair(kernel_size)
    sh, sw = pair(kernel_size if stride is None else stride)
    ph, pw = pair(padding)
    n, c, h, w = x.shape
    return (n, c, h, w, kh, kw, sh, sw, ph, pw)


@_reg("cuda", "max_pool2d")
def cuda_max_pool2d(x, kernel_size, stride, padding):
    _f32(x)
    env = _env(x)
    a = _pool_args(x, kernel_size, stride, padding)
    n, c, h, w, kh, kw, sh, sw, ph, pw = a
    oh, ow = (2 * ph + h - kh) // sh + 1, (2 * pw + w - kw) // sw + 1
    y = _new((n, c, oh, ow), x)
    mask = CudaMemory(x.device.index, 2 * _numel(y.shape)) if kh * kw <= 16 else None
    env.lib.max_pool2d_forward_f32(*a, _ptr(x), _ptr(y), mask.ptr if mask else None, env.stream())
    y._pool_tiemask = mask  # uint16 per output element, channels-last like y
    return y


@_reg("cuda", "max_pool2d_backward")
def cuda_max_pool2d_backward(output_grad, output, x, kernel_size, stride, padding):
    env = _env(x)
    a = _pool_args(x, kernel_size, stride, padding)
    dx = _new(x.shape, x)
    mask = getattr(output, "_pool_tiemask", None)
    env.lib.max_pool2d_backward_f32(*a, _ptr(output_grad), mask.ptr if mask else None, _ptr(output), _ptr(x), _ptr(dx), env.stream())
    return [dx]


def max_pool2d_argmax(output):
    """Window-local index (kh*KW + kw) of the first maximum for every output element, as a host
    uint8 array in logical [N,C,OH,OW] order.  Derived from the tie mask written by forward."""
    env = _env(output)
    mask = getattr(output, "_pool_tiemask", None)
    if mask is None:
        raise RuntimeError("this tensor was not produced by max_pool2d with a window of at most 16 elements")
    n, c, oh, ow = output.shape
    total = n * c * oh * ow
    arg = CudaMemory(output.device.index, total)
    env.lib.max_pool2d_argmax_u8(mask.ptr, arg.ptr, total, env.stream())
    return arg.read((n, oh, ow, c), np.uint8).transpose(0, 3, 1, 2).copy()


# ---------------------------------------------------------------------------- elementwise

@_reg("cuda", "relu")
def cuda_relu(x):
    _f32(x)
    env = _env(x)
    y = _new(x.shape, x)
    env.lib.relu_forward_f32(_ptr(x), _ptr(y), _numel(x.shape), env.stream())
    return y


@_reg("cuda", "relu_backward")
def cuda_relu_backward(output_grad, x):
    env = _env(x)
    dx = _new(x.shape, x)
    env.lib.relu_backward_f32(_ptr(output_grad), _ptr(x), _ptr(dx), _numel(x.shape), env.stream())
    return [dx]


@_reg("cuda", "add_relu")
def cuda_add_relu(x, y):
    """max(0, x + y) for same-shape operands (residual connection followed by ReLU)."""
    _f32(x, y)
    if x.shape != y.shape:
        from mytorch_b200.tensor import MismatchShapesError

        raise MismatchShapesError([x.shape, y.shape])
    env = _env(x)
    z = _new(x.shape, x)
    env.lib.add_relu_f32(_ptr(x), _ptr(y), _ptr(z), _numel(x.shape), env.stream())
    return z


@_reg("cuda", "add_relu_backward")
def cuda_add_relu_backward(output_grad, x, y):
    env = _env(x)
    g = _new(x.shape, x)
    env.lib.add_relu_backward_f32(_ptr(output_grad), _ptr(x), _ptr(y), _ptr(g), _numel(x.shape), env.stream())
    return g, g  # one tensor serves both operands: gradients are never modified in place


@_reg("cuda", "fill")
def cuda_fill(x, value):
    env = _env(x)
    if x.dtype is float32:
        env.lib.fill_f32(_ptr(x), _numel(x.shape), float(value), env.stream())
    else:
        x._native_array.write(np.full(x.shape, value, dtype=x.dtype.np_dtype))


def _host_random(x, array):
    cuda_upload(x, array.astype(x.dtype.np_dtype))


@_reg("cuda", "uniform")
def cuda_uniform(x, seed, a, b):
    # Initialisation only: drawn on the host with the reference CPU recipe, then uploaded, so a
    # model initialised on the GPU has the same weights as one initialised on the CPU.
    np.random.seed(seed)
    _host_random(x, np.random.uniform(low=a, high=b, size=x.shape))


@_reg("cuda", "normal")
def cuda_normal(x, seed, mean, stddev):
    np.random.seed(seed)
    _host_random(x, np.random.normal(mean, stddev, x.shape))


@_reg("cuda", "copy")
def cuda_copy(dst, src):
    env = _env(dst)
    if dst.shape != src.shape:
        from mytorch_b200.tensor import MismatchShapesError

        raise MismatchShapesError([dst.shape, src.shape])
    if dst.dtype is float32:
        env.lib.copy_f32(_ptr(dst), _ptr(src), _numel(dst.shape), env.stream())
    else:
        dst._native_array.copy_from(src._native_array, dst._native_array.nbytes)


@_reg("cuda", "cast")
def cuda_cast(x, dtype):
    env = _env(x)
    from mytorch_b200.dtype import int8

    kinds = {(int32, int64): 0, (int64, float32): 1, (float32, int64): 2, (int8, float32): 3}
    kind = kinds.get((x.dtype, dtype))
    if kind is None:
        raise RuntimeError(f"cast from {x.dtype} to {dtype} is not available on the cuda backend")
    if x._nhwc or (len(x.shape) == 4 and dtype is float32):
        raise RuntimeError("cast of 4-D tensors between float32 and integer types is not available on the cuda backend")
    out = _new(x.shape, x, dtype)
    env.lib.cast(kind, _ptr(x), _ptr(out), _numel(x.shape), env.stream())
    return out


# ---------------------------------------------------------------------------- broadcast binary ops

_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "pow": 4, "pow_dx": 6, "pow_dy": 7}


def _bstrides(t, out_shape):
    """Strides of ``t`` along the dimensions of ``out_shape`` (0 where ``t`` broadcasts)."""
    pad = len(out_shape) - len(t.shape)
    st = _strides(t)
    return [0] * pad + [0 if t.shape[i] == 1 and out_shape[pad + i] != 1 else st[i] for i in range(len(t.shape))]


def _binary(name, x, y, alpha=1.0):
    _f32(x, y)
    env = _env(x)
    shape = calculate_broadcast_shape(x.shape, y.shape)
    z = _new(shape, x)
    n = _numel(shape)
    if x.shape == y.shape and name in ("add", "sub", "mul"):
        if name == "mul":
            env.lib.mul_f32(_ptr(x), _ptr(y), _ptr(z), n, env.stream())
        else:
            env.lib.add_f32(_ptr(x), _ptr(y), _ptr(z), n, float(alpha) if name == "add" else -float(alpha), env.stream())
        return z
    if name == "add" and len(x.shape) == 2 and y.shape == (x.shape[1],):
        env.lib.add_bias_rows_f32(_ptr(x), _ptr(y), _ptr(z), x.shape[0], x.shape[1], float(alpha), env.stream())
        return z
    env.lib.binary_strided_f32(_OPS[name], len(shape), _ll(shape), _ll(_bstrides(x, shape)), _ll(_bstrides(y, shape)),
                               _ll(_strides(z)), _ptr(x), _ptr(y), _ptr(z), float(alpha), env.stream())
    return z


def _scaled(t, scale):
    if scale == 1:
        return t
    env = _env(t)
    out = _new(t.shape, t)
    env.lib.scale_f32(_ptr(out), _ptr(t), _numel(t.shape), float(scale), env.stream())
    return out


def _reduce_to(g, shape, like):
    """Sum ``g`` over the dimensions along which a tensor of ``shape`` was broadcast."""
    if tuple(g.shape) == tuple(shape):
        return g
    pad = len(g.shape) - len(shape)
    dims = tuple(i for i in range(len(g.shape)) if i < pad or (shape[i - pad] == 1 and g.shape[i] != 1))
    out = cuda_sum_scale(g, dims, True, 1)
    return cuda_reshape(out, shape)


@_reg("cuda", "add")
def cuda_add(x, y, alpha):
    return _binary("add", x, y, alpha)


@_reg("cuda", "sub")
def cuda_sub(x, y, alpha):
    return _binary("sub", x, y, alpha)


@_reg("cuda", "mul")
def cuda_mul(x, y):
    return _binary("mul", x, y)


@_reg("cuda", "div")
def cuda_div(x, y):
    return _binary("div", x, y)


@_reg("cuda", "pow")
def cuda_pow(x, y):
    return _binary("pow", x, y)


@_reg("cuda", "add_backward")
def cuda_add_backward(output_grad, x, y, alpha):
    # Same-shape operands receive the upstream gradient itself (no copy): nothing mutates
    # gradients in place, accumulation always writes a fresh tensor.
    return _reduce_to(output_grad, x.shape, x), _reduce_to(_scaled(output_grad, alpha), y.shape, y)


@_reg("cuda", "sub_backward")
def cuda_sub_backward(output_grad, x, y, alpha):
    return _reduce_to(output_grad, x.shape, x), _reduce_to(_scaled(output_grad, -alpha), y.shape, y)


@_reg("cuda", "mul_backward")
def cuda_mul_backward(output_grad, x, y):
    return _reduce_to(_binary("mul", output_grad, y), x.shape, x), _reduce_to(_binary("mul", output_grad, x), y.shape, y)


@_reg("cuda", "div_backward")
def cuda_div_backward(output_grad, x, y):
    """dx = dy / y, dy_ = -x / y^2 * dy (``mytorch/backends/cpu/ops/broadcast_binary_ops.py:108-115``)."""
    gx = _binary("div", output_grad, y)
    gy = _scaled(_binary("div", _binary("mul", output_grad, x), _binary("mul", y, y)), -1.0)
    return _reduce_to(gx, x.shape, x), _reduce_to(gy, y.shape, y)


@_reg("cuda", "pow_backward")
def cuda_pow_backward(output_grad, x, y):
    """dx = y x^(y-1) dy, dy_ = x^y ln(x) dy (``mytorch/backends/cpu/ops/broadcast_binary_ops.py:130-137``)."""
    gx = _binary("mul", _binary("pow_dx", x, y), output_grad)
    gy = _binary("mul", _binary("pow_dy", x, y), output_grad)
    return _reduce_to(gx, x.shape, x), _reduce_to(gy, y.shape, y)


# ---------------------------------------------------------------------------- max / eq / bmm

@_reg("cuda", "max")
def cuda_max(tensor, dim, keepdim):
    """(values, int64 indices) of the maximum along ``dim`` (``None``: over everything, index into the
    flattened logical tensor); ties go to the first element (``mytorch/backends/cuda/ops/max.py:10-75``)."""
    _f32(tensor)
    if dim is not None and not isinstance(dim, int):
        raise RuntimeError(f"max dimension must be a integer or None: {dim}")
    env = _env(tensor)
    nd = len(tensor.shape)
    src = tensor
    if dim is None:
        if _nontrivial_nhwc(tensor):  # flat indices refer to the logical order
            src = cuda_reshape(tensor, (_numel(tensor.shape),))
        kept_shape, kept_strides, red_len, red_stride = [], [], _numel(tensor.shape), 1
        out_shape = calculate_reduce_shape(tensor.shape, tuple(range(nd)), keepdim)
    else:
        dim = dim + nd if dim < 0 else dim
        st = _strides(tensor)
        kept = [i for i in range(nd) if i != dim]
        kept_shape, kept_strides = [tensor.shape[i] for i in kept], [st[i] for i in kept]
        red_len, red_stride = tensor.shape[dim], st[dim]
        out_shape = calculate_reduce_shape(tensor.shape, (dim,), keepdim)
    n_out = _numel(out_shape)
    values = _T()(shape=(n_out,), dtype=tensor.dtype, device=tensor.device)
    indices = _T()(shape=tuple(out_shape), dtype=int64, device=tensor.device)
    env.lib.max_strided_f32(_ptr(src), _ptr(values), _ptr(indices), len(kept_shape), _ll(kept_shape), _ll(kept_strides), red_len, red_stride,
                            env.stream())
    return cuda_reshape(values, tuple(out_shape)), indices


@_reg("cuda", "max_backward")
def cuda_max_backward(output_grad, indices_tensor, tensor, dim, keepdim):
    env = _env(tensor)
    nd = len(tensor.shape)
    dx = _new(tensor.shape, tensor)
    g = output_grad
    if _nontrivial_nhwc(g):  # the kernel reads dy in logical (dense) order, like the indices
        g = cuda_reshape(g, (_numel(g.shape),))
    if dim is None:
        flat = _T()(shape=(_numel(tensor.shape),), dtype=tensor.dtype, device=tensor.device)
        env.lib.max_backward_f32(_ptr(g), _ptr(indices_tensor), _ptr(flat), _numel(tensor.shape), 0, _ll([]), _ll([]), 1, env.stream())
        return [cuda_reshape(flat, tensor.shape)]
    dim = dim + nd if dim < 0 else dim
    st = _strides(dx)
    kept = [i for i in range(nd) if i != dim]
    env.lib.max_backward_f32(_ptr(g), _ptr(indices_tensor), _ptr(dx), _numel(tensor.shape), len(kept), _ll([tensor.shape[i] for i in kept]),
                             _ll([st[i] for i in kept]), st[dim], env.stream())
    return [dx]


@_reg("cuda", "eq")
def cuda_eq(x, y):
    """int8 tensor of element-wise equality (``mytorch/backends/cuda/ops/eq.py:9``)."""
    from mytorch_b200.dtype import int8
    from mytorch_b200.tensor import InvalidDataTypeError, MismatchShapesError

    if x.shape != y.shape:
        raise MismatchShapesError([x.shape, y.shape])
    kinds = {float32: 0, int64: 1}
    if x.dtype not in kinds or y.dtype is not x.dtype:
        raise InvalidDataTypeError(x.dtype)
    env = _env(x)
    out = _T()(shape=x.shape, dtype=int8, device=x.device)
    env.lib.eq_strided(kinds[x.dtype], len(x.shape), _ll(x.shape), _ll(_strides(x)), _ll(_strides(y)), _ptr(x), _ptr(y), _ptr(out), env.stream())
    return out


def _bmm_into(env, batch, m, n, k, a, ta, b, tb, c):
    """c[i] = op(a[i]) op(b[i]) for i < batch; dense 3-D operands, one GEMM per batch entry."""
    sa, sb, sc = 4 * (a.shape[1] * a.shape[2]), 4 * (b.shape[1] * b.shape[2]), 4 * m * n
    for i in range(batch):
        env.lib.gemm_f32(m, n, k, _ptr(a) + i * sa, ta, _ptr(b) + i * sb, tb, None, 0, _ptr(c) + i * sc, env.stream())


@_reg("cuda", "bmm")
def cuda_bmm(x, y):
    """[B,M,K] x [B,K,N] -> [B,M,N] (``mytorch/backends/cuda/ops/mm.py:131-138``)."""
    _f32(x, y)
    from mytorch_b200.tensor import MismatchShapesError

    if len(x.shape) != 3 or len(y.shape) != 3 or x.shape[0] != y.shape[0] or x.shape[2] != y.shape[1]:
        raise MismatchShapesError([x.shape, y.shape])
    env = _env(x)
    bsz, m, k = x.shape
    n = y.shape[2]
    z = _new((bsz, m, n), x)
    _bmm_into(env, bsz, m, n, k, x, 0, y, 0, z)
    return z


@_reg("cuda", "bmm_backward")
def cuda_bmm_backward(output_grad, x, y):
    env = _env(x)
    bsz, m, k = x.shape
    n = y.shape[2]
    dx, dy = _new(x.shape, x), _new(y.shape, y)
    _bmm_into(env, bsz, m, k, n, output_grad, 0, y, 1, dx)   # dx[i] = dz[i] y[i]^T
    _bmm_into(env, bsz, k, n, m, x, 1, output_grad, 0, dy)   # dy[i] = x[i]^T dz[i]
    return dx, dy


# ---------------------------------------------------------------------------- reductions

@_reg("cuda", "sum_scale")
def cuda_sum_scale(x, dim, keepdim, scale):
    _f32(x)
    env = _env(x)
    dim = tuple(dim)
    out_shape = calculate_reduce_shape(x.shape, dim, keepdim)
    out = _new(out_shape, x)
    st = env.stream()
    if x._nhwc and dim == (2, 3):
        n, c, h, w = x.shape
        env.lib.nhwc_spatial_sum_f32(_ptr(x), _ptr(out), n, c, h * w, float(scale), st)
        return out
    if x._nhwc and dim == (0, 2, 3):
        n, c, h, w = x.shape
        ws, ws_bytes = env.workspace(env.lib.colsum_workspace_bytes(c))
        env.lib.colsum_f32(_ptr(x), n * h * w, c, float(scale), _ptr(out), ws, ws_bytes, st)
        return out
    xs = _strides(x)
    kept = [i for i in range(len(x.shape)) if i not in dim]
    red = list(dim)
    dense = out if not _nontrivial_nhwc(out) else _T()(shape=(_numel(out_shape),), dtype=x.dtype, device=x.device)
    env.lib.sum_strided_f32(_ptr(x), _ptr(dense), len(kept), _ll([x.shape[i] for i in kept]), _ll([xs[i] for i in kept]),
                            len(red), _ll([x.shape[i] for i in red]), _ll([xs[i] for i in red]), float(scale), st)
    if dense is not out:
        n, c, h, w = out_shape
        env.lib.nchw_to_nhwc_f32(_ptr(dense), _ptr(out), n, c, h, w, st)
    return out


@_reg("cuda", "sum_scale_backward")
def cuda_sum_scale_backward(output_grad, x, dim, keepdim, scale):
    env = _env(x)
    dim = tuple(dim)
    dx = _new(x.shape, x)
    st = env.stream()
    if x._nhwc and dim == (2, 3):
        n, c, h, w = x.shape
        env.lib.nhwc_spatial_bcast_f32(_ptr(output_grad), _ptr(dx), n, c, h * w, float(scale), st)
        return [dx]
    gs = _strides(output_grad)
    if keepdim:
        src = [0 if i in dim else gs[i] for i in range(len(x.shape))]
    else:
        it = iter(gs)
        src = [0 if i in dim else next(it) for i in range(len(x.shape))]
    env.lib.binary_strided_f32(5, len(x.shape), _ll(x.shape), _ll(src), _ll(src), _ll(_strides(dx)), _ptr(output_grad), None,
                               _ptr(dx), float(scale), st)
    return [dx]


# ---------------------------------------------------------------------------- shape ops

def _dense_copy(env, t):
    """Logical row-major copy of a channels-last tensor."""
    n, c, h, w = t.shape
    out = CudaMemory(t.device.index, t._native_array.nbytes)
    env.lib.nhwc_to_nchw_f32(_ptr(t), out.ptr, n, c, h, w, env.stream())
    return out


@_reg("cuda", "reshape")
def cuda_reshape(x, shape):
    from mytorch_b200.tensor import channels_last

    env = _env(x)
    new_shape = calculate_reshaped_shape(x.shape, shape)
    out = _T()(tensor=x)
    out.shape = tuple(new_shape)
    out._nhwc = channels_last(out.shape, out.dtype, "cuda")
    mem = x._native_array
    if _nontrivial_nhwc(x):
        mem = _dense_copy(env, x)
    if _nontrivial_nhwc(out):
        n, c, h, w = out.shape
        dst = CudaMemory(x.device.index, mem.nbytes)
        env.lib.nchw_to_nhwc_f32(mem.ptr, dst.ptr, n, c, h, w, env.stream())
        mem = dst
    out._native_array = mem
    return out


@_reg("cuda", "permute")
def cuda_permute(x, dims):
    _f32(x)
    env = _env(x)
    out = _new([x.shape[d] for d in dims], x)
    xs = _strides(x)
    src = [xs[d] for d in dims]
    env.lib.binary_strided_f32(5, len(dims), _ll(out.shape), _ll(src), _ll(src), _ll(_strides(out)), _ptr(x), None, _ptr(out), 1.0,
                               env.stream())
    return out


@_reg("cuda", "permute_backward")
def cuda_permute_backward(output_grad, x, dims):
    inverse = [0] * len(dims)
    for i, d in enumerate(dims):
        inverse[d] = i
    return [cuda_permute(output_grad, tuple(inverse))]


# ---------------------------------------------------------------------------- loss

@_reg("cuda", "cross_entropy")
def cuda_cross_entropy(input, target):
    from mytorch_b200.tensor import InvalidDataTypeError

    if target.dtype is not int64:
        raise InvalidDataTypeError(target.dtype)
    _f32(input)
    env = _env(input)
    b, c = input.shape
    loss = _new((1,), input)
    ws, ws_bytes = env.workspace(env.lib.cross_entropy_workspace_bytes(b))
    env.lib.cross_entropy_forward_f32(b, c, _ptr(input), _ptr(target), _ptr(loss), ws, ws_bytes, env.stream())
    return loss


@_reg("cuda", "cross_entropy_backward")
def cuda_cross_entropy_backward(output_grad, input, target):
    env = _env(input)
    b, c = input.shape
    dx = _new(input.shape, input)
    env.lib.cross_entropy_backward_f32(b, c, _ptr(input), _ptr(target), _ptr(output_grad), _ptr(dx), env.stream())
    return [dx]


# ---------------------------------------------------------------------------- optimiser

def _refuse_first_step_in_capture(env, is_first_time):
    """A captured first step would bake "momentum buffer = gradient" into the graph and every replay
    would reset the momentum; the momentum buffers must exist (one eager step) before capture."""
    if is_first_time and env.capturing():
        raise RuntimeError("optimizer state does not exist yet: run one eager optimizer step before capturing the step in a CUDA graph")


@_reg("cuda", "sgd")
def cuda_sgd(param, momentum_buffer, is_first_time, lr, weight_decay, momentum, dampening, nesterov, maximize):
    env = _env(param)
    _refuse_first_step_in_capture(env, is_first_time)
    env.lib.sgd_f32(_ptr(param), _ptr(param.grad), _ptr(momentum_buffer), _numel(param.shape), int(bool(is_first_time)), float(lr),
                    float(weight_decay), float(momentum), float(dampening), int(bool(nesterov)), int(bool(maximize)), 1.0, env.stream())


@_reg("cuda", "sgd_multi")
def cuda_sgd_multi(entries, lr, weight_decay, momentum, dampening, nesterov, maximize, grad_scale=1.0):
    """entries: [(param, momentum_buffer, is_first_time)]; one launch per 96 tensors."""
    if not entries:
        return
    env = _env(entries[0][0])
    _refuse_first_step_in_capture(env, any(f for _, _, f in entries))
    k = len(entries)
    vp = ctypes.c_void_p
    params = (vp * k)(*[_ptr(p) for p, _, _ in entries])
    grads = (vp * k)(*[_ptr(p.grad) for p, _, _ in entries])
    bufs = (vp * k)(*[_ptr(b) for _, b, _ in entries])
    sizes = (_LL * k)(*[_numel(p.shape) for p, _, _ in entries])
    first = (ctypes.c_int * k)(*[int(bool(f)) for _, _, f in entries])
    env.lib.sgd_multi_f32(k, params, grads, bufs, sizes, first, float(lr), float(weight_decay), float(momentum), float(dampening),
                          int(bool(nesterov)), int(bool(maximize)), float(grad_scale), env.stream())
