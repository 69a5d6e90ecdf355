"""The NumPy oracle against fixtures produced by the reference's own CPU backend."""
import numpy as np

from conftest import load_golden, rel_err, summarize
from oracle import models, ops
from oracle import ops as O

TOL = 2e-6  # both sides are fp32 results of float64/fp32 NumPy arithmetic


def test_conv_matches_reference():
    g = load_golden("conv")
    for i in range(int(g["count"])):
        n, ci, h, w, co, k, s, p, bias = g[f"c{i}_cfg"]
        x, wt, dy = g[f"c{i}_x"], g[f"c{i}_w"], g[f"c{i}_dy"]
        b = g[f"c{i}_b"] if bias else None
        y = ops.conv2d_forward(x, wt, b, (s, s), (p, p))
        assert y.dtype == np.float32 and rel_err(y, g[f"c{i}_y"]) < TOL
        dx, dw, db = ops.conv2d_backward(dy, x, wt, bool(bias), (s, s), (p, p))
        assert rel_err(dx, g[f"c{i}_dx"]) < TOL
        assert rel_err(dw, g[f"c{i}_dw"]) < TOL
        if bias:
            assert rel_err(db, g[f"c{i}_db"]) < TOL


def test_batch_norm_matches_reference():
    g = load_golden("batch_norm")
    for i in range(int(g["count"])):
        x, gm, b, rm, rv, dy = (g[f"b{i}_{k}"] for k in ("x", "g", "b", "rm", "rv", "dy"))
        y, mean, var, rm2, rv2 = ops.batch_norm2d_forward(x, gm, b, 1e-5, True, 0.1, rm, rv)
        assert rel_err(y, g[f"b{i}_y"]) < TOL
        assert rel_err(rm2, g[f"b{i}_rm2"]) < TOL and rel_err(rv2, g[f"b{i}_rv2"]) < TOL
        dx, dg, db = ops.batch_norm2d_backward(dy, mean, var, x, gm, 1e-5)
        assert rel_err(dx, g[f"b{i}_dx"]) < 1e-5
        assert rel_err(dg, g[f"b{i}_dg"]) < 1e-5 and rel_err(db, g[f"b{i}_db"]) < 1e-5
        ye = ops.batch_norm2d_forward(x, gm, b, 1e-5, False, 0.1, rm, rv)[0]
        assert rel_err(ye, g[f"b{i}_yeval"]) < TOL


def test_max_pool_matches_reference_bit_exact():
    g = load_golden("max_pool")
    for i in range(int(g["count"])):
        k, s, p, _ = g[f"p{i}_cfg"]
        x, dy = g[f"p{i}_x"], g[f"p{i}_dy"]
        y = ops.max_pool2d_forward(x, k, s, p)
        assert np.array_equal(y, g[f"p{i}_y"])
        dx = ops.max_pool2d_backward(dy, y, x, k, s, p)
        assert rel_err(dx, g[f"p{i}_dx"]) < TOL
        am = ops.max_pool2d_argmax(x, k, s, p)
        mask = ops.max_pool2d_tiemask(x, k, s, p)
        assert np.array_equal(mask & -mask, 1 << am)  # lowest tied bit is the argmax


def test_misc_ops_match_reference():
    g = load_golden("misc")
    assert np.array_equal(ops.relu_forward(g["relu_x"]), g["relu_y"])
    assert np.array_equal(ops.relu_backward(g["relu_dy"], g["relu_x"]), g["relu_dx"])
    assert np.array_equal(ops.add_forward(g["add_a"], g["add_b"]), g["add_y"])
    da, db = ops.add_backward(g["add_dy"], g["add_a"].shape, g["add_b"].shape)
    assert np.array_equal(da, g["add_da"]) and np.array_equal(db, g["add_db"])
    assert np.array_equal(ops.add_forward(g["badd_a"], g["badd_b"]), g["badd_y"])
    da, db = ops.add_backward(g["badd_dy"], g["badd_a"].shape, g["badd_b"].shape)
    assert np.array_equal(da, g["badd_da"]) and rel_err(db, g["badd_db"]) < TOL
    y = ops.sum_scale_forward(g["gap_x"], (2, 3), False, 1 / 16)
    assert rel_err(y, g["gap_y"]) < TOL
    assert rel_err(ops.sum_scale_backward(g["gap_dy"], g["gap_x"].shape, (2, 3), False, 1 / 16), g["gap_dx"]) < TOL
    assert rel_err(ops.sum_scale_forward(g["gap_x"], (0, 2, 3), False, 1), g["csum_y"]) < TOL
    assert rel_err(ops.sum_scale_backward(g["csum_dy"], g["gap_x"].shape, (0, 2, 3), False, 1), g["csum_dx"]) < TOL
    y = ops.linear_forward(g["lin_x"], g["lin_w"], g["lin_b"])
    assert rel_err(y, g["lin_y"]) < TOL
    dx, dw, db = ops.linear_backward(g["lin_dy"], g["lin_x"], g["lin_w"], True)
    assert rel_err(dx, g["lin_dx"]) < TOL and rel_err(dw, g["lin_dw"]) < TOL and rel_err(db, g["lin_db"]) < TOL
    assert rel_err(ops.cross_entropy_forward(g["ce_z"], g["ce_t"]), g["ce_loss"]) < TOL
    assert rel_err(ops.cross_entropy_backward(np.ones((), np.float32), g["ce_z"], g["ce_t"]), g["ce_dz"]) < TOL


def test_sgd_matches_reference():
    g = load_golden("misc")
    cfgs = [dict(lr=0.1, momentum=0.9), dict(lr=0.05, momentum=0.8, nesterov=True, weight_decay=1e-2),
            dict(lr=0.01, momentum=0.5, dampening=0.3, maximize=True)]
    for i, kw in enumerate(cfgs):
        p, buf = ops.sgd_step(g[f"sgd{i}_p0"], g[f"sgd{i}_g1"], None, True, **kw)
        assert rel_err(p, g[f"sgd{i}_p1"]) < TOL
        p, buf = ops.sgd_step(p.astype(np.float32), g[f"sgd{i}_g2"], buf, False, **kw)
        assert rel_err(p, g[f"sgd{i}_p2"]) < TOL and rel_err(buf, g[f"sgd{i}_buf"]) < TOL


def test_seeded_init_matches_reference():
    g = load_golden("misc")
    s = models.SeedStream(77)
    c = models.Conv(s, 3, 4, 3)
    l = models.Linear(s, 6, 5)
    assert np.array_equal(c.w, g["init_cw"]) and np.array_equal(c.b, g["init_cb"])
    assert np.array_equal(l.w, g["init_lw"]) and np.array_equal(l.b, g["init_lb"])


def _check_summary(g, prefix, named, tol):
    for name, arr in named:
        stats, sample = summarize(arr)
        ref = g[f"{prefix}/{name}/sample"]
        scale = max(np.max(np.abs(ref)), 1e-30)
        assert np.max(np.abs(sample - ref)) / scale < tol, (prefix, name)
        assert abs(stats[2] - g[f"{prefix}/{name}/stats"][2]) <= tol * max(g[f"{prefix}/{name}/stats"][2], 1e-30), (prefix, name)


def _run_model(g, tag, net, x, t, lr, momentum, steps, tol=2e-5):
    _check_summary(g, f"{tag}/init", [(n, getattr(l, a)) for n, l, a in net.named_params()], 1e-7)
    for s in range(steps):
        loss, grads = net.train_step(x, t, lr, momentum)
        assert abs(loss - g[f"{tag}/losses"][s]) < 1e-5 * abs(g[f"{tag}/losses"][s])
        _check_summary(g, f"{tag}/grad{s}", list(grads.items()), tol)
        _check_summary(g, f"{tag}/param{s}", [(n, getattr(l, a)) for n, l, a in net.named_params()], tol)


def test_small_cnn_steps_match_reference():
    g = load_golden("models")
    rng = np.random.default_rng(1000)
    x = rng.standard_normal((64, 1, 28, 28)).astype(np.float32)
    t = rng.integers(0, 10, 64).astype(np.int64)
    _run_model(g, "cnn", models.small_cnn(1000), x, t, 0.01, 0.9, 2)


def test_resnet18_steps_match_reference():
    g = load_golden("models")
    rng = np.random.default_rng(1003)
    x = rng.standard_normal((8, 3, 32, 32)).astype(np.float32)
    t = rng.integers(0, 10, 8).astype(np.int64)
    _run_model(g, "resnet_w8", models.resnet18_cifar(1003, (8, 16, 32, 64)), x, t, 0.1, 0.9, 2, tol=1e-4)
    rng = np.random.default_rng(1004)
    x = rng.standard_normal((4, 3, 32, 32)).astype(np.float32)
    t = rng.integers(0, 10, 4).astype(np.int64)
    _run_model(g, "resnet_full", models.resnet18_cifar(1004), x, t, 0.1, 0.9, 1, tol=1e-4)


def test_bn_relu_pool_block_matches_reference():
    g = load_golden("models")
    rng = np.random.default_rng(1002)
    x = (0.5 + 2.0 * rng.standard_normal((8, 16, 12, 12))).astype(np.float32)
    dy = rng.standard_normal((8, 16, 6, 6)).astype(np.float32)
    r = models.bn_relu_pool_block(x, dy, 16)
    assert rel_err(r["y"], g["block/y"]) < TOL
    assert rel_err(r["dx"], g["block/dx"]) < 1e-5
    assert rel_err(r["dgamma"], g["block/dgamma"]) < 1e-5 and rel_err(r["dbeta"], g["block/dbeta"]) < 1e-5
    assert rel_err(r["running_mean"], g["block/rm"]) < TOL and rel_err(r["running_var"], g["block/rv"]) < TOL


def test_operators_beside_the_training_step_match_reference():
    """div / pow gradients, bmm, eq, max along a dimension and BatchNorm1d of the oracle against fixtures
    written by the reference's CPU backend (tests/golden/make_golden.py, ``extra_op_cases``)."""
    gd = load_golden("extra_ops")
    for i in range(3):
        for name, fwd, bwd in (("div", lambda a, b: a / b, O.div_backward), ("pow", np.power, O.pow_backward)):
            x, y, dz = gd[f"{name}{i}_x"], gd[f"{name}{i}_y"], gd[f"{name}{i}_dz"]
            assert rel_err(fwd(x, y), gd[f"{name}{i}_z"]) < 1e-6
            dx, dy = bwd(dz, x, y)
            assert dx.shape == x.shape and dy.shape == y.shape
            assert rel_err(dx, gd[f"{name}{i}_dx"]) < 1e-5 and rel_err(dy, gd[f"{name}{i}_dy"]) < 1e-5
    assert rel_err(O.bmm_forward(gd["bmm_x"], gd["bmm_y"]), gd["bmm_z"]) < 1e-6
    dx, dy = O.bmm_backward(gd["bmm_dz"], gd["bmm_x"], gd["bmm_y"])
    assert rel_err(dx, gd["bmm_dx"]) < 1e-6 and rel_err(dy, gd["bmm_dy"]) < 1e-6
    assert np.array_equal(O.eq_forward(gd["eq_a"], gd["eq_b"]), gd["eq_z"])
    for dim in (0, 1, 2):
        v, i = O.max_forward(gd["max_x"], dim, False)
        assert np.array_equal(v, gd[f"max{dim}_v"]) and np.array_equal(i, gd[f"max{dim}_i"])
    for i in range(2):
        x, dy = gd[f"bn1d{i}_x"], gd[f"bn1d{i}_dy"]
        x4 = x.reshape(x.shape[0], 12, -1, 1)
        ones, zeros = np.ones(12, np.float32), np.zeros(12, np.float32)
        y, mean, var, rm, rv = O.batch_norm2d_forward(x4, ones, zeros, 1e-5, True, 0.1, zeros, ones)
        dx, dg, db = O.batch_norm2d_backward(dy.reshape(x4.shape), mean, var, x4, ones, 1e-5)
        assert rel_err(y.reshape(x.shape), gd[f"bn1d{i}_y"]) < 1e-5 and rel_err(dx.reshape(x.shape), gd[f"bn1d{i}_dx"]) < 2e-5
        assert rel_err(dg, gd[f"bn1d{i}_dg"]) < 2e-5 and rel_err(db, gd[f"bn1d{i}_db"]) < 2e-5
        assert rel_err(rm, gd[f"bn1d{i}_rm"]) < 1e-5 and rel_err(rv, gd[f"bn1d{i}_rv"]) < 1e-5
