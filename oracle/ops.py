"""CPU oracle for the CNN training-step operators (TEST INFRASTRUCTURE ONLY).

This module is a NumPy restatement of the reference's CPU backend
(``mytorch/backends/cpu/ops/*.py`` in tigert1998/mytorch).  It exists so that the
CUDA kernels can be checked on machines where the reference itself is not
present.  Only the test-suite, the smoke check and the benchmark's CPU-baseline
leg may import it; the product package never does.

Parity status: the reference ships no tests, golden vectors or fixtures of its own.
The oracle is pinned against outputs of the reference's CPU backend executed in the
build container (``tests/golden/*.npz``, produced by ``tests/golden/make_golden.py``).

All arrays are logical NCHW / row-major, exactly as the reference's tensors.
Each function cites the reference file:line it restates.
"""
from __future__ import annotations

import numpy as np
from numpy.lib.stride_tricks import sliding_window_view


def round_tf32(a):
    """float32 values rounded to TF32 (10 mantissa bits, round to nearest, ties to even), returned as
    float32.  No counterpart in the reference, whose GPU kernels multiply in fp32: this models the one
    place where the tensor-core kernels deviate from fp32 arithmetic.  Their operands pass through
    tensor maps of type TFLOAT32, and the copy engine rounds them this way on the way into shared
    memory (measured: results agree with this model to 1e-5, against 3e-4 for unrounded operands and
    9e-4 for truncation); products and sums are then exact / fp32.  Feeding rounded operands to the
    functions below therefore predicts the tensor-core results up to fp32 accumulation error."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0xFFF + ((u >> 13) & 1)) & 0xFFFFE000
    return u.astype(np.uint32).view(np.float32).reshape(a.shape)


def _pair(v):
    return (int(v), int(v)) if np.isscalar(v) else tuple(int(i) for i in v)


def conv_out_hw(h, w, kh, kw, stride, padding):
    """Output extent rule, mytorch/backends/cpu/ops/conv.py:16-17."""
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    return (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1


def _im2col(x, kh, kw, stride, padding):
    """Patch matrix [N*OH*OW, C*KH*KW] in float64 with (c, kh, kw) column order.

    mytorch/backends/cpu/ops/conv.py:9-39 — the reference's buffer is ``np.zeros`` of the
    default dtype, so every convolution GEMM on CPU runs in float64.
    """
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    n, c, h, w = x.shape
    oh, ow = conv_out_hw(h, w, kh, kw, stride, padding)
    xp = np.pad(x, [(0, 0), (0, 0), (ph, ph), (pw, pw)])
    win = sliding_window_view(xp, (kh, kw), axis=(2, 3))  # n c H' W' kh kw
    win = win[:, :, : (oh - 1) * sh + 1 : sh, : (ow - 1) * sw + 1 : sw]
    col = np.ascontiguousarray(win.transpose(0, 2, 3, 1, 4, 5), dtype=np.float64)
    return col.reshape(n * oh * ow, c * kh * kw)


def conv2d_forward(x, w, b, stride, padding):
    """mytorch/backends/cpu/ops/conv.py:76-97: float64 GEMM + bias, rounded to x.dtype."""
    n = x.shape[0]
    cout, _, kh, kw = w.shape
    oh, ow = conv_out_hw(x.shape[2], x.shape[3], kh, kw, stride, padding)
    y = _im2col(x, kh, kw, stride, padding) @ w.reshape(cout, -1).T
    if b is not None:
        y += b
    return y.reshape(n, oh, ow, cout).transpose(0, 3, 1, 2).astype(x.dtype)


def conv2d_backward(dy, x, w, has_bias, stride, padding):
    """mytorch/backends/cpu/ops/conv.py:100-133.

    dX: the [M, Cin*KH*KW] product is rounded to x.dtype and then scatter-added in a
    float64 image (``_col2im``, conv.py:42-73), so dX is float64 like the reference's.
    dW: patchesᵀ·dY rounded to w.dtype.  db: column sums of dY (dY's dtype).
    """
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    n, cin, h, wd = x.shape
    cout, _, kh, kw = w.shape
    oh, ow = conv_out_hw(h, wd, kh, kw, stride, padding)
    dy_mat = dy.transpose(0, 2, 3, 1).reshape(-1, cout)
    col = _im2col(x, kh, kw, stride, padding)
    dcol = (dy_mat @ w.reshape(cout, -1)).astype(x.dtype)
    dcol = dcol.reshape(n, oh, ow, cin, kh, kw).transpose(0, 3, 4, 5, 1, 2)
    img = np.zeros((n, cin, h + 2 * ph + sh - 1, wd + 2 * pw + sw - 1))
    for i in range(kh):
        for j in range(kw):
            img[:, :, i : i + sh * oh : sh, j : j + sw * ow : sw] += dcol[:, :, i, j]
    dx = img[:, :, ph : h + ph, pw : wd + pw]
    dw = (dy_mat.T @ col).astype(w.dtype).reshape(w.shape)
    db = dy_mat.sum(axis=0) if has_bias else None
    return dx, dw, db


def linear_forward(x, w, b):
    """nn/linear.py:59-65 on backends/cpu/ops/mm.py:6-11: x·Wᵀ (+ b) in x.dtype."""
    y = np.matmul(x, w.T)
    if b is not None:
        y = y + b
    return y


def linear_backward(dy, x, w, has_bias):
    """backends/cpu/ops/mm.py:14-22 composed with the permute/add backward of Linear:
    dX = dY·W, dW = (Xᵀ·dY)ᵀ, db = Σ_rows dY (broadcast_binary_ops.py:21-33)."""
    dx = np.matmul(dy, w)
    dw = np.matmul(x.T, dy).T
    db = dy.sum(axis=0) if has_bias else None
    return dx, dw, db


def batch_norm2d_forward(x, gamma, beta, eps, training, momentum, running_mean, running_var):
    """mytorch/backends/cpu/ops/batch_norm.py:10-53.

    Returns (y, mean[1,C,1,1], var[1,C,1,1], new_running_mean, new_running_var).  The
    running variance receives the *biased* batch variance (batch_norm.py:36-38).
    """
    c = x.shape[1]
    axes = (0, 2, 3)
    new_rm, new_rv = running_mean, running_var
    if training:
        mean = x.mean(axis=axes, keepdims=True)
        var = x.var(axis=axes, keepdims=True, ddof=0)
        if running_mean is not None and running_var is not None:
            one_m = np.asarray(1 - momentum, dtype=x.dtype)
            mom = np.asarray(momentum, dtype=x.dtype)
            new_rm = one_m * running_mean + mom * mean.reshape(c)
            new_rv = one_m * running_var + mom * var.reshape(c)
    else:
        if running_mean is not None and running_var is not None:
            mean = running_mean.reshape(1, c, 1, 1)
            var = running_var.reshape(1, c, 1, 1)
        else:
            mean = x.mean(axis=axes, keepdims=True)
            var = x.var(axis=axes, keepdims=True, ddof=0)
    xhat = (x - mean) / np.sqrt(var + eps)
    if gamma is not None and beta is not None:
        y = gamma.reshape(1, c, 1, 1) * xhat + beta.reshape(1, c, 1, 1)
    else:
        y = xhat
    return y, mean, var, new_rm, new_rv


def batch_norm2d_backward(dy, mean, var, x, gamma, eps):
    """mytorch/backends/cpu/ops/batch_norm.py:56-98 (dx, dgamma, dbeta)."""
    c = x.shape[1]
    axes = (0, 2, 3)
    m = x.shape[0] * x.shape[2] * x.shape[3]
    xhat = (x - mean) / np.sqrt(var + eps)
    if gamma is not None:
        dbeta = dy.sum(axes, dtype=x.dtype)
        dgamma = (dy * xhat).sum(axes, dtype=x.dtype)
        dxhat = dy * gamma.reshape(1, c, 1, 1)
    else:
        dbeta = dgamma = None
        dxhat = dy
    dvar = (dxhat * -0.5 * (x - mean) * (var + eps) ** -1.5).sum(axis=axes, keepdims=True)
    dmean = (dxhat * -((var + eps) ** -0.5)).sum(axis=axes, keepdims=True)
    dx = dxhat * (var + eps) ** -0.5
    dx += dmean / m
    dx += dvar * 2 / m * (x - mean)
    return dx, dgamma, dbeta


def _pool_windows(x, kernel_size, stride, padding):
    kh, kw = _pair(kernel_size)
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    n, c, h, w = x.shape
    oh = (2 * ph + h - kh) // sh + 1
    ow = (2 * pw + w - kw) // sw + 1
    xp = np.pad(x, ((0, 0), (0, 0), (ph, ph), (pw, pw)))  # padded cells hold 0, not -inf
    win = sliding_window_view(xp, (kh, kw), axis=(2, 3))
    win = win[:, :, : (oh - 1) * sh + 1 : sh, : (ow - 1) * sw + 1 : sw]
    return xp, win, oh, ow


def max_pool2d_forward(x, kernel_size, stride, padding):
    """mytorch/backends/cpu/ops/pool_ops.py:7-47.  Padding cells take part with value 0."""
    _, win, _, _ = _pool_windows(x, kernel_size, stride, padding)
    return win.max(axis=(4, 5))


def max_pool2d_argmax(x, kernel_size, stride, padding):
    """First maximal element of each window in row-major (kh, kw) order, as an index
    kh*KW+kw.  The reference keeps no index tensor; this is ``np.argmax`` over the very
    window view its forward reduces (pool_ops.py:24-44)."""
    _, win, _, _ = _pool_windows(x, kernel_size, stride, padding)
    flat = win.reshape(*win.shape[:4], -1)
    return flat.argmax(axis=-1).astype(np.int64)


def max_pool2d_tiemask(x, kernel_size, stride, padding):
    """Bit kh*KW+kw is set where the window element equals the window maximum
    (the ``input_windows == output`` mask of pool_ops.py:91-96)."""
    _, win, _, _ = _pool_windows(x, kernel_size, stride, padding)
    flat = win.reshape(*win.shape[:4], -1)
    eq = flat == flat.max(axis=-1, keepdims=True)
    bits = (1 << np.arange(flat.shape[-1], dtype=np.int64))
    return (eq * bits).sum(axis=-1)


def max_pool2d_backward(dy, out, x, kernel_size, stride, padding):
    """mytorch/backends/cpu/ops/pool_ops.py:50-115: every window element equal to the
    window maximum receives the window's gradient; overlapping windows accumulate."""
    kh, kw = _pair(kernel_size)
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    xp, win, oh, ow = _pool_windows(x, kernel_size, stride, padding)
    gw = (win == out[..., None, None]) * dy[..., None, None]
    gp = np.zeros_like(xp)
    for i in range(oh):
        for j in range(ow):
            gp[:, :, i * sh : i * sh + kh, j * sw : j * sw + kw] += gw[:, :, i, j]
    h, w = x.shape[2], x.shape[3]
    return gp[:, :, ph : ph + h, pw : pw + w]


def relu_forward(x):
    """mytorch/backends/cpu/ops/elementwise_ops.py:25-31."""
    return np.maximum(x, 0)


def relu_backward(dy, x):
    """mytorch/backends/cpu/ops/elementwise_ops.py:34-41: gradient is blocked only where
    x < 0 (at x == 0 it passes, unlike the reference's CUDA kernel)."""
    dx = dy.copy()
    dx[x < 0] = 0
    return dx


def add_forward(x, y, alpha=1):
    """mytorch/backends/cpu/ops/broadcast_binary_ops.py:36-45."""
    return x + y * alpha


def _reduce_to(g, shape):
    extra = g.ndim - len(shape)
    padded = (1,) * extra + tuple(shape)
    axes = tuple(i for i in range(g.ndim) if padded[i] != g.shape[i])
    return g.sum(axis=axes).reshape(shape)


def add_backward(dy, x_shape, y_shape, alpha=1):
    """mytorch/backends/cpu/ops/broadcast_binary_ops.py:11-33, :48-53."""
    return _reduce_to(dy, x_shape), _reduce_to(dy * alpha, y_shape)


def mul_forward(x, y):
    """mytorch/backends/cpu/ops/broadcast_binary_ops.py:76-85."""
    return x * y


def mul_backward(dy, x, y):
    """mytorch/backends/cpu/ops/broadcast_binary_ops.py:88-93."""
    return _reduce_to(y * dy, x.shape), _reduce_to(x * dy, y.shape)


def sum_scale_forward(x, dim, keepdim, scale):
    """mytorch/backends/cpu/ops/reduce_ops.py:7-17."""
    return np.sum(x, axis=tuple(dim), keepdims=keepdim) * scale


def sum_scale_backward(dy, x_shape, dim, keepdim, scale):
    """mytorch/backends/cpu/ops/reduce_ops.py:20-34."""
    g = dy * scale if keepdim else np.expand_dims(dy, tuple(dim)) * scale
    return np.broadcast_to(g, x_shape).copy()


def _softmax(z):
    """mytorch/backends/cpu/ops/cross_entropy.py:8-12."""
    z = z - np.max(z, axis=1, keepdims=True)
    e = np.exp(z)
    return e / np.sum(e, axis=1, keepdims=True)


def cross_entropy_forward(logits, target):
    """mytorch/backends/cpu/ops/cross_entropy.py:15-29: mean of -log softmax[target]."""
    sm = _softmax(logits)
    nll = -np.log(sm[np.arange(logits.shape[0]), target])
    return np.array(np.mean(nll), dtype=logits.dtype)


def cross_entropy_backward(dy, logits, target):
    """mytorch/backends/cpu/ops/cross_entropy.py:32-47."""
    b, c = logits.shape
    onehot = np.eye(c, dtype=logits.dtype)[target]
    return (_softmax(logits) - onehot) * dy / b


def sgd_step(param, grad, buf, is_first, lr, weight_decay=0.0, momentum=0.0,
             dampening=0.0, nesterov=False, maximize=False):
    """mytorch/backends/cpu/ops/sgd.py:5-29.  Returns (new_param, new_buf).  The momentum
    buffer is set to g on the first step and the momentum path runs even for momentum 0."""
    g = -grad if maximize else grad
    g = g + weight_decay * param
    buf = g if is_first else (momentum * buf + (1 - dampening) * g)
    g = (g + momentum * buf) if nesterov else buf
    return param - g * lr, buf


def uniform_init(shape, seed, a, b, dtype=np.float32):
    """mytorch/backends/cpu/ops/elementwise_ops.py:17-22 (global NumPy seed, then uniform)."""
    np.random.seed(seed)
    return np.random.uniform(low=a, high=b, size=shape).astype(dtype)


# ---------------------------------------------------------------------------- operators beside the training step

def div_backward(dy, x, y):
    """mytorch/backends/cpu/ops/broadcast_binary_ops.py:108-115 (with the reductions of _backward_cpu, :21-33)."""
    return _reduce_to(1 / y * dy, x.shape), _reduce_to(-x / (y ** 2) * dy, y.shape)


def pow_backward(dy, x, y):
    """mytorch/backends/cpu/ops/broadcast_binary_ops.py:130-137."""
    return _reduce_to(y * np.power(x, y - 1) * dy, x.shape), _reduce_to(np.power(x, y) * np.log(x) * dy, y.shape)


def max_forward(x, dim, keepdim):
    """mytorch/backends/cpu/ops/max.py:7-23: values and, for an integer ``dim``, int64 argmax indices
    (first maximum).  With ``dim=None`` the CUDA backend (mytorch/backends/cuda/ops/max.py:15-16) reduces
    over every dimension and records the index into the flattened tensor."""
    values = np.max(x, axis=dim, keepdims=keepdim).astype(x.dtype)
    if dim is None:
        return values, np.argmax(x).astype(np.int64).reshape(values.shape)
    return values, np.argmax(x, axis=dim, keepdims=keepdim).astype(np.int64)


def max_backward(dy, indices, x_shape, dim, keepdim):
    """mytorch/backends/cuda/ops/max.py:75-120: the gradient goes to the recorded index, zeros elsewhere."""
    dx = np.zeros(x_shape, dtype=dy.dtype)
    if dim is None:
        dx.reshape(-1)[int(np.asarray(indices).reshape(-1)[0])] = np.asarray(dy).reshape(-1)[0]
        return dx
    idx = indices if keepdim else np.expand_dims(indices, dim)
    g = dy if keepdim else np.expand_dims(dy, dim)
    np.put_along_axis(dx, idx, g, axis=dim)
    return dx


def eq_forward(x, y):
    """mytorch/backends/cpu/ops/eq.py:9-19."""
    return (x == y).astype(np.int8)


def bmm_forward(x, y):
    """mytorch/backends/cpu/ops/mm.py:26-31."""
    return np.matmul(x, y)


def bmm_backward(dy, x, y):
    """mytorch/backends/cpu/ops/mm.py:34-47."""
    return np.matmul(dy, np.transpose(y, (0, 2, 1))), np.matmul(np.transpose(x, (0, 2, 1)), dy)
