"""Generate golden fixtures by running the reference's own CPU backend.

Run from the repository root in a container that has the reference checked out:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

The script imports the reference package ``mytorch`` from the given path (never from this
repository), drives its public API on seeded inputs and writes ``tests/golden/*.npz``.
Those files are the only thing that travels: the tests never need the reference.
"""
import os
import sys

import numpy as np

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MYTORCH_REFERENCE", "")
if not REF or not os.path.isdir(os.path.join(REF, "mytorch")):
    sys.exit("usage: make_golden.py <path to a tigert1998/mytorch checkout>")
sys.path.insert(0, REF)

import mytorch  # noqa: E402  (the reference)
import mytorch.nn as nn  # noqa: E402
import mytorch.nn.functional as F  # noqa: E402
from mytorch.nn.functional.batch_norm import _batch_norm2d  # noqa: E402
from mytorch.optim import SGD  # noqa: E402
from mytorch.rand_generator import manual_seed  # noqa: E402
from mytorch.tensor import Tensor  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
f32 = np.float32


def T(a, grad=False):
    return Tensor(cpu_array=np.ascontiguousarray(a), requires_grad=grad)


def npy(t):
    return None if t is None else np.asarray(t._cpu_array)


def backward_with(y, dy):
    (y * T(dy)).sum().backward()


def conv_cases():
    out = {}
    cases = [  # n cin h w cout k s p bias
        (2, 3, 9, 9, 8, 3, 1, 1, True),
        (2, 4, 8, 8, 8, 3, 2, 1, False),
        (1, 8, 7, 7, 16, 1, 2, 0, False),
        (2, 1, 10, 10, 4, 3, 1, 0, True),
        (2, 16, 12, 12, 32, 3, 1, 1, True),
        (1, 4, 11, 13, 8, 5, 2, 2, True),
        (3, 32, 8, 8, 64, 3, 1, 1, False),
    ]
    rng = np.random.default_rng(11)
    for i, (n, ci, h, w, co, k, s, p, bias) in enumerate(cases):
        x = rng.standard_normal((n, ci, h, w)).astype(f32)
        wt = (rng.standard_normal((co, ci, k, k)) / np.sqrt(ci * k * k)).astype(f32)
        b = rng.standard_normal(co).astype(f32) if bias else None
        xt, wtt = T(x, True), T(wt, True)
        bt = T(b, True) if bias else None
        y = F.conv2d(xt, wtt, bt, s, p)
        dy = rng.standard_normal(y.shape).astype(f32)
        backward_with(y, dy)
        out[f"c{i}_cfg"] = np.array([n, ci, h, w, co, k, s, p, int(bias)])
        out[f"c{i}_x"], out[f"c{i}_w"], out[f"c{i}_dy"] = x, wt, dy
        if bias:
            out[f"c{i}_b"] = b
            out[f"c{i}_db"] = npy(bt.grad)
        out[f"c{i}_y"], out[f"c{i}_dx"], out[f"c{i}_dw"] = npy(y), npy(xt.grad), npy(wtt.grad)
    out["count"] = np.array(len(cases))
    np.savez_compressed(os.path.join(OUT, "conv.npz"), **out)


def bn_cases():
    out = {}
    rng = np.random.default_rng(12)
    shapes = [(4, 8, 6, 6), (3, 5, 7, 5), (8, 16, 4, 4)]
    for i, shp in enumerate(shapes):
        c = shp[1]
        x = (0.5 + 2.0 * rng.standard_normal(shp)).astype(f32)
        g = rng.uniform(0.5, 1.5, c).astype(f32)
        b = rng.standard_normal(c).astype(f32)
        rm, rv = rng.standard_normal(c).astype(f32), rng.uniform(0.5, 2, c).astype(f32)
        xt, gt, bt, rmt, rvt = T(x, True), T(g, True), T(b, True), T(rm.copy()), T(rv.copy())
        y = _batch_norm2d(xt, gt, bt, 1e-5, True, 0.1, rmt, rvt)
        dy = rng.standard_normal(shp).astype(f32)
        backward_with(y, dy)
        ye = _batch_norm2d(T(x), T(g), T(b), 1e-5, False, 0.1, T(rm.copy()), T(rv.copy()))
        out.update({f"b{i}_x": x, f"b{i}_g": g, f"b{i}_b": b, f"b{i}_rm": rm, f"b{i}_rv": rv,
                    f"b{i}_dy": dy, f"b{i}_y": npy(y), f"b{i}_rm2": npy(rmt), f"b{i}_rv2": npy(rvt),
                    f"b{i}_dx": npy(xt.grad), f"b{i}_dg": npy(gt.grad), f"b{i}_db": npy(bt.grad),
                    f"b{i}_yeval": npy(ye)})
    out["count"] = np.array(len(shapes))
    np.savez_compressed(os.path.join(OUT, "batch_norm.npz"), **out)


def pool_cases():
    out = {}
    rng = np.random.default_rng(13)
    cases = [  # shape k s p ties
        ((2, 4, 8, 8), 2, 2, 0, False),
        ((2, 4, 9, 9), 3, 2, 1, False),
        ((1, 3, 7, 7), 2, 1, 0, False),
        ((2, 4, 8, 8), 2, 2, 0, True),
        ((2, 8, 6, 6), 3, 1, 1, True),
        ((2, 4, 6, 6), 2, 2, 1, False),
    ]
    for i, (shp, k, s, p, ties) in enumerate(cases):
        if ties:
            x = rng.integers(-2, 3, shp).astype(f32)
        else:
            x = rng.standard_normal(shp).astype(f32)
        xt = T(x, True)
        y = F.max_pool2d(xt, (k, k), (s, s), (p, p))
        dy = rng.standard_normal(y.shape).astype(f32)
        backward_with(y, dy)
        out.update({f"p{i}_cfg": np.array([k, s, p, int(ties)]), f"p{i}_x": x, f"p{i}_dy": dy,
                    f"p{i}_y": npy(y), f"p{i}_dx": npy(xt.grad)})
    out["count"] = np.array(len(cases))
    np.savez_compressed(os.path.join(OUT, "max_pool.npz"), **out)


def misc_cases():
    out = {}
    rng = np.random.default_rng(14)
    # relu (with exact zeros)
    x = rng.standard_normal((3, 4, 5, 5)).astype(f32)
    x[0, 0, 0, :3] = 0
    xt = T(x, True)
    y = F.relu(xt)
    dy = rng.standard_normal(x.shape).astype(f32)
    backward_with(y, dy)
    out.update(relu_x=x, relu_dy=dy, relu_y=npy(y), relu_dx=npy(xt.grad))
    # add: same shape (alpha 1) and row broadcast
    a, b = rng.standard_normal((2, 3, 4, 4)).astype(f32), rng.standard_normal((2, 3, 4, 4)).astype(f32)
    at, bt = T(a, True), T(b, True)
    y = at + bt
    dy = rng.standard_normal(a.shape).astype(f32)
    backward_with(y, dy)
    out.update(add_a=a, add_b=b, add_dy=dy, add_y=npy(y), add_da=npy(at.grad), add_db=npy(bt.grad))
    a, b = rng.standard_normal((6, 10)).astype(f32), rng.standard_normal((10,)).astype(f32)
    at, bt = T(a, True), T(b, True)
    y = at + bt
    dy = rng.standard_normal(a.shape).astype(f32)
    backward_with(y, dy)
    out.update(badd_a=a, badd_b=b, badd_dy=dy, badd_y=npy(y), badd_da=npy(at.grad), badd_db=npy(bt.grad))
    # sum_scale: global average pool and a (0,2,3) sum
    x = rng.standard_normal((3, 6, 4, 4)).astype(f32)
    xt = T(x, True)
    y = xt.mean(dim=(2, 3))
    dy = rng.standard_normal(y.shape).astype(f32)
    backward_with(y, dy)
    out.update(gap_x=x, gap_dy=dy, gap_y=npy(y), gap_dx=npy(xt.grad))
    xt = T(x, True)
    y = xt.sum(dim=(0, 2, 3))
    dy = rng.standard_normal(y.shape).astype(f32)
    backward_with(y, dy)
    out.update(csum_dy=dy, csum_y=npy(y), csum_dx=npy(xt.grad))
    # linear (through the reference's nn.Linear: reshape, permute, mm, add, reshape)
    manual_seed(5)
    lin = nn.Linear(20, 7)
    x = rng.standard_normal((9, 20)).astype(f32)
    xt = T(x, True)
    y = lin(xt)
    dy = rng.standard_normal(y.shape).astype(f32)
    backward_with(y, dy)
    out.update(lin_x=x, lin_w=npy(lin.weight), lin_b=npy(lin.bias), lin_dy=dy, lin_y=npy(y),
               lin_dx=npy(xt.grad), lin_dw=npy(lin.weight.grad), lin_db=npy(lin.bias.grad))
    # cross entropy
    z = (3 * rng.standard_normal((8, 10))).astype(f32)
    t = rng.integers(0, 10, 8).astype(np.int64)
    zt = T(z, True)
    loss = F.cross_entropy(zt, T(t))
    loss.backward()
    out.update(ce_z=z, ce_t=t, ce_loss=npy(loss), ce_dz=npy(zt.grad))
    # sgd: two steps for three hyper-parameter sets
    for i, kw in enumerate([dict(lr=0.1, momentum=0.9), dict(lr=0.05, momentum=0.8, nesterov=True, weight_decay=1e-2),
                            dict(lr=0.01, momentum=0.5, dampening=0.3, maximize=True)]):
        p0 = rng.standard_normal((5, 7)).astype(f32)
        g1, g2 = rng.standard_normal((5, 7)).astype(f32), rng.standard_normal((5, 7)).astype(f32)
        p = nn.Parameter(T(p0.copy()))
        opt = SGD([p], **kw)
        p.grad = T(g1.copy())
        opt.step()
        p1 = npy(p).copy()
        p.grad = T(g2.copy())
        opt.step()
        out.update({f"sgd{i}_p0": p0, f"sgd{i}_g1": g1, f"sgd{i}_g2": g2, f"sgd{i}_p1": p1,
                    f"sgd{i}_p2": npy(p).copy(), f"sgd{i}_buf": npy(opt.state[p]["momentum_buffer"]).copy()})
    # seeded init of two layers (pins the RNG restatement)
    manual_seed(77)
    c = nn.Conv2d(3, 4, 3)
    l = nn.Linear(6, 5)
    out.update(init_cw=npy(c.weight), init_cb=npy(c.bias), init_lw=npy(l.weight), init_lb=npy(l.bias))
    np.savez_compressed(os.path.join(OUT, "misc.npz"), **out)


class BasicBlock(nn.Module):
    def __init__(self, cin, cout, stride):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(cout)
        self.conv2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(cout)
        self.downsample = None
        if stride != 1 or cin != cout:
            self.downsample = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, 0, bias=False), nn.BatchNorm2d(cout))
        self.relu = nn.ReLU()

    def forward(self, x):
        y = self.bn2(self.conv2(self.relu(self.bn1(self.conv1(x)))))
        sc = x if self.downsample is None else self.downsample(x)
        return self.relu(y + sc)


class ResNet18(nn.Module):
    def __init__(self, widths, num_classes=10):
        super().__init__()
        self.conv1 = nn.Conv2d(3, widths[0], 3, 1, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(widths[0])
        self.relu = nn.ReLU()
        cin = widths[0]
        for si, wd in enumerate(widths):
            blocks = []
            for bi in range(2):
                blocks.append(BasicBlock(cin, wd, 2 if (si > 0 and bi == 0) else 1))
                cin = wd
            setattr(self, f"layer{si + 1}", nn.Sequential(*blocks))
        self.fc = nn.Linear(cin, num_classes)

    def forward(self, x):
        x = self.relu(self.bn1(self.conv1(x)))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(x.mean(dim=(2, 3)))


def summarize(prefix, named, out, sample=64):
    for name, arr in named:
        a = np.asarray(arr, dtype=np.float64).reshape(-1)
        idx = np.linspace(0, a.size - 1, min(sample, a.size)).astype(np.int64)
        out[f"{prefix}/{name}/stats"] = np.array([a.sum(), np.abs(a).sum(), np.sqrt((a * a).sum())])
        out[f"{prefix}/{name}/sample"] = a[idx]


def train_steps(model, x, t, lr, momentum, steps, out, tag):
    opt = SGD(model.parameters(), lr=lr, momentum=momentum)
    summarize(f"{tag}/init", [(k, npy(v)) for k, v in model.named_parameters()], out)
    losses = []
    for s in range(steps):
        loss = F.cross_entropy(model(T(x)), T(t))
        opt.zero_grad()
        loss.backward()
        summarize(f"{tag}/grad{s}", [(k, npy(v.grad)) for k, v in model.named_parameters()], out)
        opt.step()
        summarize(f"{tag}/param{s}", [(k, npy(v)) for k, v in model.named_parameters()], out)
        losses.append(loss.item())
    summarize(f"{tag}/buffers", [(k, npy(v)) for k, v in model.named_buffers()], out)
    out[f"{tag}/losses"] = np.array(losses)


def model_cases():
    out = {}
    # small CNN of the MNIST-shaped configuration, full size (batch 64), 2 steps
    rng = np.random.default_rng(1000)
    x = rng.standard_normal((64, 1, 28, 28)).astype(f32)
    t = rng.integers(0, 10, 64).astype(np.int64)
    manual_seed(1000)

    class Flat(nn.Module):
        def forward(self, x):
            return x.reshape((x.shape[0], -1))

    net = nn.Sequential(nn.Conv2d(1, 32, 3), nn.ReLU(), nn.Conv2d(32, 64, 3), nn.ReLU(), nn.MaxPool2d(2, 2),
                        Flat(), nn.Linear(9216, 128), nn.ReLU(), nn.Linear(128, 10))
    train_steps(net, x, t, 0.01, 0.9, 2, out, "cnn")
    # ResNet-18 (CIFAR variant) at reduced widths and batch, 2 steps
    rng = np.random.default_rng(1003)
    x = rng.standard_normal((8, 3, 32, 32)).astype(f32)
    t = rng.integers(0, 10, 8).astype(np.int64)
    manual_seed(1003)
    train_steps(ResNet18((8, 16, 32, 64)), x, t, 0.1, 0.9, 2, out, "resnet_w8")
    # ResNet-18 at full widths, batch 4, one step (pins the real channel counts)
    rng = np.random.default_rng(1004)
    x = rng.standard_normal((4, 3, 32, 32)).astype(f32)
    t = rng.integers(0, 10, 4).astype(np.int64)
    manual_seed(1004)
    train_steps(ResNet18((64, 128, 256, 512)), x, t, 0.1, 0.9, 1, out, "resnet_full")
    # BN -> ReLU -> MaxPool block
    rng = np.random.default_rng(1002)
    x = (0.5 + 2.0 * rng.standard_normal((8, 16, 12, 12))).astype(f32)
    dy = rng.standard_normal((8, 16, 6, 6)).astype(f32)
    bn = nn.BatchNorm2d(16)
    xt = T(x, True)
    y = nn.MaxPool2d(2, 2)(nn.ReLU()(bn(xt)))
    backward_with(y, dy)
    out.update({"block/y": npy(y), "block/dx": npy(xt.grad), "block/dgamma": npy(bn.weight.grad),
                "block/dbeta": npy(bn.bias.grad), "block/rm": npy(bn.running_mean), "block/rv": npy(bn.running_var)})
    np.savez_compressed(os.path.join(OUT, "models.npz"), **out)


def _shard_bounds(n, rank, world):
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def sharded_step(build, seed, x, t, world, lr, momentum, out, tag, want_grads=True):
    """Data parallelism emulated with the reference itself: every shard of the batch runs through
    the same initial weights (BatchNorm therefore sees the statistics of its shard only), the
    shard gradients are averaged, and one SGD step is taken with the average.  The reported loss
    is the mean of the shard losses.  With world == 1 this is the plain reference step."""
    losses, sums = [], None
    for r in range(world):
        lo, hi = _shard_bounds(x.shape[0], r, world)
        manual_seed(seed)
        model = build()
        loss = F.cross_entropy(model(T(x[lo:hi])), T(t[lo:hi]))
        losses.append(loss.item())
        if not want_grads:
            continue
        loss.backward()
        grads = [(k, np.asarray(npy(v.grad), dtype=np.float64)) for k, v in model.named_parameters()]
        sums = grads if sums is None else [(k, a + b) for (k, a), (_, b) in zip(sums, grads)]
    out[f"{tag}/shard_losses"] = np.array(losses)
    out[f"{tag}/loss"] = np.array(float(np.mean(losses)))
    if not want_grads:
        return
    avg = [(k, (a / world).astype(f32)) for k, a in sums]
    summarize(f"{tag}/grad", avg, out)
    manual_seed(seed)
    model = build()
    opt = SGD(model.parameters(), lr=lr, momentum=momentum)
    for (k, p), (_, g) in zip(model.named_parameters(), avg):
        p.grad = T(g)
    opt.step()
    summarize(f"{tag}/param", [(k, npy(v)) for k, v in model.named_parameters()], out)


def dp_cases():
    """Sharded data-parallel steps: a reduced-width ResNet-18 on 2 and 4 shards with gradients, and the
    benchmark configuration (full-width ResNet-18, batch 512, seed 1003) with gradients on 1 shard
    and first-step losses on 2, 4 and 8 shards."""
    out = {}
    rng = np.random.default_rng(2002)
    x = rng.standard_normal((16, 3, 32, 32)).astype(f32)
    t = rng.integers(0, 10, 16).astype(np.int64)
    for world in (2, 4):
        sharded_step(lambda: ResNet18((16, 32, 64, 64)), 2002, x, t, world, 0.1, 0.9, out, f"dp_small/w{world}")
    rng = np.random.default_rng(1003)
    x = rng.standard_normal((512, 3, 32, 32)).astype(f32)
    t = rng.integers(0, 10, 512).astype(np.int64)
    full = lambda: ResNet18((64, 128, 256, 512))
    sharded_step(full, 1003, x, t, 1, 0.1, 0.9, out, "c3_b512/w1")
    for world in (2, 4, 8):
        sharded_step(full, 1003, x, t, world, 0.1, 0.9, out, f"c3_b512/w{world}", want_grads=False)
    np.savez_compressed(os.path.join(OUT, "data_parallel.npz"), **out)


def extra_op_cases():
    """Operators beside the training step: div / pow gradients (with broadcasting), bmm, eq, max along a
    dimension, BatchNorm1d, all through the reference's public API on its CPU backend."""
    import mytorch

    out = {}
    rng = np.random.default_rng(15)
    for i, (xs, ys) in enumerate([((4, 6), (4, 6)), ((4, 6), (6,)), ((2, 3, 4, 5), (1, 3, 1, 1))]):
        x, y = rng.uniform(0.5, 2.0, xs).astype(f32), rng.uniform(0.5, 2.0, ys).astype(f32)
        dz = rng.standard_normal(np.broadcast_shapes(xs, ys)).astype(f32)
        for name, fn in (("div", lambda a, b: a / b), ("pow", lambda a, b: a ** b)):
            xt, yt = T(x, True), T(y, True)
            z = fn(xt, yt)
            backward_with(z, dz)
            out.update({f"{name}{i}_x": x, f"{name}{i}_y": y, f"{name}{i}_dz": dz, f"{name}{i}_z": npy(z),
                        f"{name}{i}_dx": npy(xt.grad), f"{name}{i}_dy": npy(yt.grad)})
    x, y = rng.standard_normal((3, 5, 7)).astype(f32), rng.standard_normal((3, 7, 6)).astype(f32)
    dz = rng.standard_normal((3, 5, 6)).astype(f32)
    xt, yt = T(x, True), T(y, True)
    z = mytorch.bmm(xt, yt)
    backward_with(z, dz)
    out.update(bmm_x=x, bmm_y=y, bmm_dz=dz, bmm_z=npy(z), bmm_dx=npy(xt.grad), bmm_dy=npy(yt.grad))
    a, b = rng.integers(0, 3, (4, 9)).astype(f32), rng.integers(0, 3, (4, 9)).astype(f32)
    out.update(eq_a=a, eq_b=b, eq_z=npy(T(a).eq(T(b))))
    m = rng.integers(-4, 5, (3, 5, 6)).astype(f32)
    for dim in (0, 1, 2):
        v, idx = T(m).max(dim, False)
        out.update({"max_x": m, f"max{dim}_v": npy(v), f"max{dim}_i": npy(idx)})
    for i, shape in enumerate([(16, 12), (6, 12, 10)]):
        x = (1.0 + rng.standard_normal(shape)).astype(f32)
        dy = rng.standard_normal(shape).astype(f32)
        bn = nn.BatchNorm1d(12)
        xt = T(x, True)
        yv = bn(xt)
        backward_with(yv, dy)
        out.update({f"bn1d{i}_x": x, f"bn1d{i}_dy": dy, f"bn1d{i}_y": npy(yv), f"bn1d{i}_dx": npy(xt.grad), f"bn1d{i}_dg": npy(bn.weight.grad),
                    f"bn1d{i}_db": npy(bn.bias.grad), f"bn1d{i}_rm": npy(bn.running_mean), f"bn1d{i}_rv": npy(bn.running_var)})
    np.savez_compressed(os.path.join(OUT, "extra_ops.npz"), **out)


def checkpoint_case():
    """A checkpoint written by the reference's own ``mytorch.save`` after one SGD-momentum step of a small
    Conv-BN-ReLU-MaxPool-Linear net (model and optimizer state dicts), and what the reference computes
    when it takes the next step from that state: the file must load into the new implementation and
    the continued step must agree."""
    import mytorch

    class Flat(nn.Module):
        def forward(self, x):
            return x.reshape((x.shape[0], -1))

    rng = np.random.default_rng(3003)
    x = rng.standard_normal((8, 3, 12, 12)).astype(f32)
    t = rng.integers(0, 5, 8).astype(np.int64)
    manual_seed(3003)
    net = nn.Sequential(nn.Conv2d(3, 8, 3, 1, 1), nn.BatchNorm2d(8), nn.ReLU(), nn.MaxPool2d(2, 2), Flat(), nn.Linear(8 * 6 * 6, 5))
    opt = SGD(net.parameters(), lr=0.05, momentum=0.9)

    def step():
        loss = F.cross_entropy(net(T(x)), T(t))
        opt.zero_grad()
        loss.backward()
        opt.step()
        return loss.item()

    out = {"loss0": np.array(step())}
    mytorch.save({"model": net.state_dict(), "optimizer": opt.state_dict()}, os.path.join(OUT, "reference_checkpoint.pt"))
    for k, v in net.state_dict().items():
        out[f"saved/{k}"] = npy(v).copy()
    for i, p in enumerate(net.parameters()):
        out[f"momentum/{i}"] = npy(opt.state[p]["momentum_buffer"]).copy()
    out["loss1"] = np.array(step())
    for k, v in net.state_dict().items():
        out[f"next/{k}"] = npy(v).copy()
    np.savez_compressed(os.path.join(OUT, "checkpoint.npz"), **out)


if __name__ == "__main__":
    only = sys.argv[2:]  # optional: names of the fixture groups to regenerate
    groups = {"conv": conv_cases, "bn": bn_cases, "pool": pool_cases, "misc": misc_cases, "models": model_cases, "dp": dp_cases, "checkpoint": checkpoint_case, "extra": extra_op_cases}
    for name, fn in groups.items():
        if not only or name in only:
            fn()
    print("golden fixtures written to", OUT)
