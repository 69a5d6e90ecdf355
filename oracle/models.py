"""CPU oracle: whole training steps composed from ``oracle.ops`` (TEST INFRASTRUCTURE ONLY).

The reference drives its operators through a tape (``mytorch/autograd.py:120-179``) and
``optim/sgd.py:28-56``.  Here the same arithmetic is laid out as explicit layer objects
with a hand-written backward, so that a full step (forward, loss, backward, SGD) can be
replayed without the reference being present.  Gradients that reach a tensor from two
consumers are added in the order the reference's tape would add them.

Seeded initialisation restates ``mytorch/rand_generator.py:4-24`` +
``mytorch/nn/init.py:10-17`` + ``nn/conv.py:63-69`` / ``nn/linear.py:52-57``: the meta seed
feeds Python's ``random``; every ``uniform_`` draws one ``randint(0, 1e9+7)`` which seeds
NumPy's global generator for that tensor.
"""
from __future__ import annotations

import math
import random

import numpy as np

from . import ops


class SeedStream:
    """mytorch/rand_generator.py:4-24."""

    def __init__(self, meta_seed):
        self._rng = random.Random()
        self._rng.seed(meta_seed)

    def next(self):
        return self._rng.randint(0, int(round(1e9 + 7)))


def _kaiming_bound(shape):
    fan_in = int(np.prod(shape[1:]))
    a = math.sqrt(5)
    return (6 / (1 + a ** 2) / fan_in) ** 0.5, fan_in


class Conv:
    def __init__(self, seeds, cin, cout, k, stride=1, padding=0, bias=True):
        shape = (cout, cin, k, k)
        bound, fan_in = _kaiming_bound(shape)
        self.w = ops.uniform_init(shape, seeds.next(), -bound, bound)
        self.b = None
        if bias:
            bb = 1 / math.sqrt(fan_in)
            self.b = ops.uniform_init((cout,), seeds.next(), -bb, bb)
        self.stride, self.padding = (stride, stride), (padding, padding)

    def params(self):
        return [("weight", "w"), ("bias", "b")] if self.b is not None else [("weight", "w")]

    def forward(self, x):
        self.x = x
        return ops.conv2d_forward(x, self.w, self.b, self.stride, self.padding)

    def backward(self, dy):
        dx, self.dw, self.db = ops.conv2d_backward(
            dy, self.x, self.w, self.b is not None, self.stride, self.padding)
        return dx


class BN:
    def __init__(self, c, eps=1e-5, momentum=0.1):
        self.w = np.ones(c, np.float32)
        self.b = np.zeros(c, np.float32)
        self.rm = np.zeros(c, np.float32)
        self.rv = np.ones(c, np.float32)
        self.eps, self.momentum = eps, momentum

    def params(self):
        return [("weight", "w"), ("bias", "b")]

    def forward(self, x):
        self.x = x
        y, self.mean, self.var, self.rm, self.rv = ops.batch_norm2d_forward(
            x, self.w, self.b, self.eps, True, self.momentum, self.rm, self.rv)
        return y

    def backward(self, dy):
        dx, self.dw, self.db = ops.batch_norm2d_backward(dy, self.mean, self.var, self.x, self.w, self.eps)
        return dx


class ReLU:
    def params(self):
        return []

    def forward(self, x):
        self.x = x
        return ops.relu_forward(x)

    def backward(self, dy):
        return ops.relu_backward(dy, self.x)


class MaxPool:
    def __init__(self, k, stride=1, padding=0):
        self.k, self.s, self.p = (k, k), (stride, stride), (padding, padding)

    def params(self):
        return []

    def forward(self, x):
        self.x = x
        self.y = ops.max_pool2d_forward(x, self.k, self.s, self.p)
        return self.y

    def backward(self, dy):
        return ops.max_pool2d_backward(dy, self.y, self.x, self.k, self.s, self.p)


class Flatten:
    def params(self):
        return []

    def forward(self, x):
        self.shape = x.shape
        return x.reshape(x.shape[0], -1)

    def backward(self, dy):
        return dy.reshape(self.shape)


class GlobalAvgPool:
    """x.mean(dim=(2,3)) = sum_scale with scale 1/(H*W) (mytorch/ops/reduce_ops.py:36-42)."""

    def params(self):
        return []

    def forward(self, x):
        self.shape = x.shape
        self.scale = 1 / (x.shape[2] * x.shape[3])
        return ops.sum_scale_forward(x, (2, 3), False, self.scale)

    def backward(self, dy):
        return ops.sum_scale_backward(dy, self.shape, (2, 3), False, self.scale)


class Linear:
    def __init__(self, seeds, fin, fout, bias=True):
        bound, fan_in = _kaiming_bound((fout, fin))
        self.w = ops.uniform_init((fout, fin), seeds.next(), -bound, bound)
        self.b = None
        if bias:
            bb = 1 / math.sqrt(fan_in)
            self.b = ops.uniform_init((fout,), seeds.next(), -bb, bb)

    def params(self):
        return [("weight", "w"), ("bias", "b")] if self.b is not None else [("weight", "w")]

    def forward(self, x):
        self.x = x
        return ops.linear_forward(x, self.w, self.b)

    def backward(self, dy):
        dx, self.dw, self.db = ops.linear_backward(dy, self.x, self.w, self.b is not None)
        return dx


class BasicBlock:
    """conv3x3-BN-ReLU-conv3x3-BN (+ 1x1 conv-BN shortcut when the shape changes), add, ReLU."""

    def __init__(self, seeds, cin, cout, stride):
        self.conv1 = Conv(seeds, cin, cout, 3, stride, 1, bias=False)
        self.bn1 = BN(cout)
        self.relu1 = ReLU()
        self.conv2 = Conv(seeds, cout, cout, 3, 1, 1, bias=False)
        self.bn2 = BN(cout)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = (Conv(seeds, cin, cout, 1, stride, 0, bias=False), BN(cout))
        self.relu2 = ReLU()

    def named_layers(self, prefix):
        out = [(prefix + "conv1", self.conv1), (prefix + "bn1", self.bn1),
               (prefix + "conv2", self.conv2), (prefix + "bn2", self.bn2)]
        if self.down is not None:
            out += [(prefix + "downsample.0", self.down[0]), (prefix + "downsample.1", self.down[1])]
        return out

    def forward(self, x):
        y = self.bn2.forward(self.conv2.forward(self.relu1.forward(self.bn1.forward(self.conv1.forward(x)))))
        sc = x if self.down is None else self.down[1].forward(self.down[0].forward(x))
        return self.relu2.forward(ops.add_forward(y, sc, 1))

    def backward(self, dy):
        d = self.relu2.backward(dy)
        dmain = self.conv1.backward(self.bn1.backward(self.relu1.backward(
            self.conv2.backward(self.bn2.backward(d)))))
        dsc = d if self.down is None else self.down[0].backward(self.down[1].backward(d))
        return dmain + dsc


class Net:
    """A list of (name, layer) run in sequence, with softmax cross-entropy and SGD."""

    def __init__(self, named_layers):
        self.layers = named_layers
        self.bufs = {}

    def flat_layers(self):
        out = []
        for name, layer in self.layers:
            if isinstance(layer, BasicBlock):
                out += layer.named_layers(name + ".")
            else:
                out.append((name, layer))
        return out

    def named_params(self):
        out = []
        for name, layer in self.flat_layers():
            for pname, attr in layer.params():
                out.append((f"{name}.{pname}", layer, attr))
        return out

    def forward(self, x):
        for _, layer in self.layers:
            x = layer.forward(x)
        return x

    def loss_and_grads(self, x, target):
        logits = self.forward(x)
        loss = ops.cross_entropy_forward(logits, target)
        d = ops.cross_entropy_backward(np.ones((), logits.dtype), logits, target)
        for _, layer in reversed(self.layers):
            d = layer.backward(d)
        grads = {}
        for name, layer, attr in self.named_params():
            grads[name] = getattr(layer, "d" + attr)
        return float(loss), grads, logits

    def sgd(self, grads, lr, momentum=0.0, weight_decay=0.0):
        for name, layer, attr in self.named_params():
            p = getattr(layer, attr)
            first = name not in self.bufs
            newp, buf = ops.sgd_step(p, grads[name].astype(p.dtype), self.bufs.get(name), first,
                                     lr, weight_decay, momentum)
            setattr(layer, attr, newp.astype(p.dtype))
            self.bufs[name] = buf

    def train_step(self, x, target, lr, momentum=0.0):
        loss, grads, _ = self.loss_and_grads(x, target)
        self.sgd(grads, lr, momentum)
        return loss, grads


def small_cnn(meta_seed):
    """Conv(1,32,3)-ReLU-Conv(32,64,3)-ReLU-MaxPool(2)-flatten-Linear(9216,128)-ReLU-Linear(128,10)."""
    s = SeedStream(meta_seed)
    return Net([
        ("0", Conv(s, 1, 32, 3)), ("1", ReLU()), ("2", Conv(s, 32, 64, 3)), ("3", ReLU()),
        ("4", MaxPool(2, 2)), ("5", Flatten()), ("6", Linear(s, 9216, 128)), ("7", ReLU()),
        ("8", Linear(s, 128, 10)),
    ])


def resnet18_cifar(meta_seed, widths=(64, 128, 256, 512), num_classes=10, in_ch=3):
    """3x3 stem (stride 1, no max-pool), 4 stages of 2 BasicBlocks, strides 1/2/2/2,
    global average pool, Linear."""
    s = SeedStream(meta_seed)
    layers = [("conv1", Conv(s, in_ch, widths[0], 3, 1, 1, bias=False)), ("bn1", BN(widths[0])),
              ("relu", ReLU())]
    cin = widths[0]
    for si, wd in enumerate(widths):
        for bi in range(2):
            stride = 2 if (si > 0 and bi == 0) else 1
            layers.append((f"layer{si + 1}.{bi}", BasicBlock(s, cin, wd, stride)))
            cin = wd
    layers += [("avgpool", GlobalAvgPool()), ("fc", Linear(s, cin, num_classes))]
    return Net(layers)


def bn_relu_pool_block(x, dy, c, eps=1e-5, momentum=0.1):
    """BatchNorm2d(c, train) -> ReLU -> MaxPool2d(2,2), forward and backward."""
    bn, relu, pool = BN(c, eps, momentum), ReLU(), MaxPool(2, 2)
    y = pool.forward(relu.forward(bn.forward(x)))
    dx = bn.backward(relu.backward(pool.backward(dy)))
    return {"y": y, "dx": dx, "dgamma": bn.dw, "dbeta": bn.db, "running_mean": bn.rm,
            "running_var": bn.rv, "mean": bn.mean.reshape(-1), "var": bn.var.reshape(-1),
            "argmax": ops.max_pool2d_argmax(relu.forward(bn.forward(x)), (2, 2), (2, 2), (0, 0))}
