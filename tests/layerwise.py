"""Layer-by-layer ("teacher-forced") parity inside a whole model.

While a model runs forward and backward on the GPU, every operator call is intercepted; its
inputs are downloaded, the NumPy oracle computes the same operator from those very inputs,
and outputs / returned gradients are compared.  Because both sides start from identical
inputs at every layer, the comparison is not amplified by the network depth (nor by ReLU
masks that flip under rounding), so each operator can be held to its own tolerance: 5e-3 for
the TF32 tensor-core convolutions and GEMMs against the exact oracle and 5e-5 against the oracle
evaluated on TF32-rounded operands (the arithmetic the tensor cores perform), 1e-5 for fp32
operators, bit-exact for pooling.
"""
import numpy as np

from conftest import rel_err
from oracle import ops as O

TF32_TOL = 5e-3
FP32_TOL = 2e-5
# convolutions and Linear GEMMs must in addition match one of two exact arithmetic models up to fp32
# accumulation error: fp32 operands (CUDA-core kernels) or operands rounded to TF32 (tensor-core kernels)
MODEL_TOL = 5e-5


def _h(t):
    return None if t is None else t.to("cpu")._numpy()


class LayerwiseChecker:
    def __init__(self):
        from mytorch_b200.autograd import DAGTracker

        self.tracker = DAGTracker.instance()
        self.report = []  # (phase, op, worst relative error)
        self._fused_out = {}

    def _note(self, phase, op, got, want, tol, rounded=None):
        err = rel_err(got, want)
        self.report.append((phase, op, err))
        assert err <= tol, (phase, op, err, tol)
        if rounded is not None:
            model_err = min(err, rel_err(got, rounded))
            self.report.append((phase, op + "@model", model_err))
            assert model_err <= MODEL_TOL, (phase, op, model_err, MODEL_TOL)

    # ---- forward: called from the patched add_node
    def _forward(self, name, inputs, outputs, helpers):
        y = _h(outputs[0].detach())
        if name == "conv2d":
            x, w, b, s, p = inputs
            hx, hw, hb = _h(x.detach()), _h(w.detach()), _h(b.detach()) if b is not None else None
            self._note("fwd", name, y, O.conv2d_forward(hx, hw, hb, s, p), TF32_TOL, O.conv2d_forward(O.round_tf32(hx), O.round_tf32(hw), hb, s, p))
        elif name == "linear":
            x, w, b = inputs
            hx, hw, hb = _h(x.detach()), _h(w.detach()), _h(b.detach()) if b is not None else None
            self._note("fwd", name, y, O.linear_forward(hx, hw, hb), TF32_TOL, O.linear_forward(O.round_tf32(hx), O.round_tf32(hw), hb))
        elif name in ("batch_norm2d", "batch_norm2d_relu"):
            x, g, b, eps = inputs
            ry, mean, var, _, _ = O.batch_norm2d_forward(_h(x.detach()), _h(g.detach()), _h(b.detach()), eps, True, 0.1, None, None)
            if name.endswith("relu"):
                ry = O.relu_forward(ry)
                self._fused_out[id(x)] = y
            self._note("fwd", name, y, ry, FP32_TOL)
            self._note("fwd", name + ".mean", _h(helpers[0]), mean.reshape(-1), FP32_TOL)
            self._note("fwd", name + ".var", _h(helpers[1]), var.reshape(-1), FP32_TOL)
        elif name == "batch_norm2d_add_relu":
            x, res, g, b, eps = inputs
            ry, mean, var, _, _ = O.batch_norm2d_forward(_h(x.detach()), _h(g.detach()), _h(b.detach()), eps, True, 0.1, None, None)
            ry = O.relu_forward(O.add_forward(ry, _h(res.detach()), 1))
            self._fused_out[id(x)] = y
            self._note("fwd", name, y, ry, FP32_TOL)
            self._note("fwd", name + ".mean", _h(helpers[0]), mean.reshape(-1), FP32_TOL)
            self._note("fwd", name + ".var", _h(helpers[1]), var.reshape(-1), FP32_TOL)
        elif name == "relu":
            assert np.array_equal(y, O.relu_forward(_h(inputs[0].detach())))
        elif name == "max_pool2d":
            x, k, s, p = inputs
            assert np.array_equal(y, O.max_pool2d_forward(_h(x.detach()), k, s if s is not None else k, p))
        elif name == "add":
            self._note("fwd", name, y, O.add_forward(_h(inputs[0].detach()), _h(inputs[1].detach()), inputs[2]), FP32_TOL)
        elif name == "add_relu":
            assert np.array_equal(y, O.relu_forward(O.add_forward(_h(inputs[0].detach()), _h(inputs[1].detach()), 1)))
        elif name == "sum_scale":
            x, dim, keep, scale = inputs
            self._note("fwd", name, y, O.sum_scale_forward(_h(x.detach()), dim, keep, scale), FP32_TOL)
        elif name == "cross_entropy":
            self._note("fwd", name, y.reshape(()), O.cross_entropy_forward(_h(inputs[0].detach()), _h(inputs[1])), FP32_TOL)

    # ---- backward: wraps every registered backward function
    def _backward(self, name, func):
        def wrapped(*args, **kwargs):
            kwargs.pop("defer_weight_gradient", None)  # every gradient is inspected right after its operator returns
            # read before the call: an operator may add to this tensor in place and return it
            earlier = _h(kwargs["accumulate_dx"]) if kwargs.get("accumulate_dx") is not None else None
            grads = func(*args, **kwargs)
            g = [_h(t) if t is not None and hasattr(t, "shape") else None for t in grads]
            if name == "conv2d":
                dy, x, w, b, s, p = args
                rdx, rdw, rdb = O.conv2d_backward(_h(dy), _h(x.detach()), _h(w.detach()), b is not None, s, p)
                tdx, tdw, _ = O.conv2d_backward(O.round_tf32(_h(dy)), O.round_tf32(_h(x.detach())), O.round_tf32(_h(w.detach())), False, s, p)
                if g[0] is not None:
                    # with accumulate_dx the returned dx includes that earlier gradient
                    self._note("bwd", name + ".dx", g[0], rdx if earlier is None else rdx + earlier, TF32_TOL,
                               tdx if earlier is None else tdx + earlier)
                self._note("bwd", name + ".dw", g[1], rdw, TF32_TOL, tdw)
                if b is not None:
                    self._note("bwd", name + ".db", g[2], rdb, FP32_TOL * 5)
            elif name == "linear":
                dy, x, w, b = args
                rdx, rdw, rdb = O.linear_backward(_h(dy), _h(x.detach()), _h(w.detach()), b is not None)
                tdx, tdw, _ = O.linear_backward(O.round_tf32(_h(dy)), O.round_tf32(_h(x.detach())), O.round_tf32(_h(w.detach())), False)
                if g[0] is not None:
                    self._note("bwd", name + ".dx", g[0], rdx, TF32_TOL, tdx)
                self._note("bwd", name + ".dw", g[1], rdw, TF32_TOL, tdw)
                if b is not None:
                    self._note("bwd", name + ".db", g[2], rdb, FP32_TOL * 5)
            elif name in ("batch_norm2d", "batch_norm2d_relu"):
                dy, mean, var, x, gam, b, eps = args
                c = x.shape[1]
                hm, hv, hx, hdy = _h(mean).reshape(1, c, 1, 1), _h(var).reshape(1, c, 1, 1), _h(x.detach()), _h(dy)
                if name.endswith("relu"):
                    # the reference would run relu_backward on the BatchNorm output first, which blocks
                    # the gradient only where that output is negative.  The mask is taken from the
                    # forward output recorded for this node (y > 0), plus the elements whose
                    # normalised value is exactly zero (x equal to the batch mean with beta = 0):
                    # their forward output is 0 as well, but the gradient passes.
                    hg, hb = _h(gam.detach()).reshape(1, c, 1, 1), _h(b.detach()).reshape(1, c, 1, 1)
                    pre = (hx - hm) * (hg / np.sqrt(hv + np.float32(eps), dtype=np.float32)) + hb
                    keep = (self._fused_out[id(x)] > 0) | (pre == 0)
                    hdy = np.where(keep, hdy, 0).astype(hdy.dtype)
                rdx, rdg, rdb = O.batch_norm2d_backward(hdy, hm, hv, hx, _h(gam.detach()), eps)
                self._note("bwd", name + ".dx", g[0], rdx, FP32_TOL * 2)
                self._note("bwd", name + ".dgamma", g[1], rdg, FP32_TOL * 3)
                self._note("bwd", name + ".dbeta", g[2], rdb, FP32_TOL * 3)
            elif name == "batch_norm2d_add_relu":
                dy, mean, var, x, res, gam, b, eps = args
                c = x.shape[1]
                hm, hv, hx, hdy = _h(mean).reshape(1, c, 1, 1), _h(var).reshape(1, c, 1, 1), _h(x.detach()), _h(dy)
                # the reference would run relu_backward on (BatchNorm output + residual): the gradient is
                # blocked only where that sum is negative; taken from the recorded output (y > 0) plus the
                # elements whose sum is exactly zero
                hg, hb = _h(gam.detach()).reshape(1, c, 1, 1), _h(b.detach()).reshape(1, c, 1, 1)
                pre = (hx - hm) * (hg / np.sqrt(hv + np.float32(eps), dtype=np.float32)) + hb + _h(res.detach())
                keep = (self._fused_out[id(x)] > 0) | (pre == 0)
                masked = np.where(keep, hdy, 0).astype(hdy.dtype)
                assert np.array_equal(g[1], masked)   # gradient of the added tensor
                rdx, rdg, rdb = O.batch_norm2d_backward(masked, hm, hv, hx, _h(gam.detach()), eps)
                self._note("bwd", name + ".dx", g[0], rdx, FP32_TOL * 2)
                self._note("bwd", name + ".dgamma", g[2], rdg, FP32_TOL * 3)
                self._note("bwd", name + ".dbeta", g[3], rdb, FP32_TOL * 3)
            elif name == "relu":
                assert np.array_equal(g[0], O.relu_backward(_h(args[0]), _h(args[1].detach())))
            elif name == "add_relu":
                dy, x, y = args
                want = O.relu_backward(_h(dy), O.add_forward(_h(x.detach()), _h(y.detach()), 1))
                assert np.array_equal(g[0], want) and np.array_equal(g[1], want)
            elif name == "max_pool2d":
                dy, out, x, k, s, p = args
                self._note("bwd", name, g[0], O.max_pool2d_backward(_h(dy), _h(out.detach()), _h(x.detach()), k, s if s is not None else k, p), 1e-6)
            elif name == "sum_scale":
                dy, x, dim, keep, scale = args
                self._note("bwd", name, g[0], O.sum_scale_backward(_h(dy), x.shape, dim, keep, scale), FP32_TOL)
            elif name == "cross_entropy":
                dy, z, t = args
                self._note("bwd", name, g[0], O.cross_entropy_backward(_h(dy).reshape(()), _h(z.detach()), _h(t)), FP32_TOL)
            return grads

        return wrapped

    def __enter__(self):
        self._add_node = self.tracker.add_node
        self._funcs = dict(self.tracker._backward_funcs)

        def add_node(name, inputs, outputs, helpers=None):
            self._forward(name, inputs, outputs, helpers or [])
            return self._add_node(name, inputs, outputs, helpers)

        self.tracker.add_node = add_node
        for name, f in self._funcs.items():
            self.tracker._backward_funcs[name] = self._backward(name, f)
        return self

    def __exit__(self, *exc):
        self.tracker.add_node = self._add_node
        self.tracker._backward_funcs.update(self._funcs)
        return False

    def worst(self, prefix):
        return max((e for ph, op, e in self.report if op.startswith(prefix)), default=0.0)
