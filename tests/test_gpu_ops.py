"""Per-operator parity of the CUDA kernels (through the registry and the C ABI) against the
NumPy oracle and the golden fixtures from the reference's CPU backend.

Tolerances (relative to the largest reference magnitude): fp32 CUDA-core operators 1e-5;
convolution / Linear GEMMs (TF32 tensor cores where the shape allows) 5e-3; max-pool values,
tie masks and argmax indices bit-exact.
"""
import numpy as np
import pytest

from conftest import load_golden, rel_err
from oracle import ops as O

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
TF32_TOL = 5e-3
# A convolution / GEMM result must also match ONE of two exact arithmetic models to fp32 accumulation
# error: fp32 operands (the CUDA-core kernels), or operands rounded to TF32 with exact products and
# fp32 sums (the tensor-core kernels; measured 4e-7 .. 1.2e-5 up to K = 4608).
MODEL_TOL = 5e-5


def _matches_a_model(got, exact, rounded):
    return min(rel_err(got, exact), rel_err(got, rounded)) < MODEL_TOL


@pytest.fixture(scope="module")
def g():
    import gpu_util

    return gpu_util


def _conv_check(g, x, w, b, dy, s, p, ref=None):
    xt, wt = g.dev(x, True), g.dev(w, True)
    bt = g.dev(b, True) if b is not None else None
    y = g.op("conv2d")(xt, wt, bt, (s, s), (p, p))
    dx, dw, db = g.op("conv2d_backward")(g.dev(dy), xt, wt, bt, (s, s), (p, p))
    y, dx, dw = g.host(y), g.host(dx), g.host(dw)
    ey = O.conv2d_forward(x, w, b, (s, s), (p, p))
    edx, edw, edb = O.conv2d_backward(dy, x, w, b is not None, (s, s), (p, p))
    ry, rdx, rdw, rdb = (ey, edx, edw, edb) if ref is None else ref
    assert y.shape == ry.shape
    assert rel_err(y, ry) < TF32_TOL
    assert rel_err(dx, rdx) < TF32_TOL
    assert rel_err(dw, rdw) < TF32_TOL
    if b is not None:
        assert rel_err(g.host(db), rdb) < FP32_TOL * 10
    tx, tw, tdy = O.round_tf32(x), O.round_tf32(w), O.round_tf32(dy)
    tdx, tdw, _ = O.conv2d_backward(tdy, tx, tw, False, (s, s), (p, p))
    assert _matches_a_model(y, ey, O.conv2d_forward(tx, tw, b, (s, s), (p, p)))
    assert _matches_a_model(dx, edx, tdx)
    assert _matches_a_model(dw, edw, tdw)


def test_conv_golden(g):
    gd = load_golden("conv")
    for i in range(int(gd["count"])):
        n, ci, h, w, co, k, s, p, bias = (int(v) for v in gd[f"c{i}_cfg"])
        b = gd[f"c{i}_b"] if bias else None
        ref = (gd[f"c{i}_y"], gd[f"c{i}_dx"], gd[f"c{i}_dw"], gd[f"c{i}_db"] if bias else None)
        _conv_check(g, gd[f"c{i}_x"], gd[f"c{i}_w"], b, gd[f"c{i}_dy"], s, p, ref)


@pytest.mark.parametrize("cfg", [
    # n, cin, h, w, cout, k, s, p, bias     (shapes of the ResNet / benchmark layers, small batch)
    (4, 64, 56, 56, 64, 3, 1, 1, True),
    (8, 64, 32, 32, 64, 3, 1, 1, False),
    (8, 64, 32, 32, 128, 3, 2, 1, False),
    (8, 64, 32, 32, 128, 1, 2, 0, False),
    (8, 128, 16, 16, 128, 3, 1, 1, False),
    (8, 256, 8, 8, 256, 3, 1, 1, False),
    (16, 512, 4, 4, 512, 3, 1, 1, False),
    (8, 3, 32, 32, 64, 3, 1, 1, False),
    (2, 32, 26, 26, 64, 3, 1, 0, True),
    (2, 3, 37, 41, 16, 7, 2, 3, False),
    (3, 20, 9, 11, 24, 3, 1, 1, True),
    # stride-1 "same" filters on the row-staged kernels: odd image sizes, tiles that straddle images,
    # partial channel blocks, 5x5 and 7x7 filters, more than two output-channel tiles, a row too wide
    # for the row stage (falls back to the im2col kernels)
    (3, 32, 17, 23, 40, 3, 1, 1, True),
    (2, 64, 20, 36, 64, 5, 1, 2, False),
    (2, 96, 24, 24, 72, 3, 1, 1, True),
    (1, 64, 64, 64, 192, 3, 1, 1, False),
    (4, 160, 16, 16, 128, 3, 1, 1, False),
    (2, 32, 32, 32, 32, 7, 1, 3, False),
    (1, 32, 40, 250, 32, 3, 1, 1, False),
])
def test_conv_oracle(g, cfg):
    n, ci, h, w, co, k, s, p, bias = cfg
    rng = np.random.default_rng(hash(cfg) % (2 ** 31))
    x = rng.standard_normal((n, ci, h, w)).astype(np.float32)
    wt = (rng.standard_normal((co, ci, k, k)) / np.sqrt(ci * k * k)).astype(np.float32)
    b = rng.standard_normal(co).astype(np.float32) if bias else None
    oh, ow = O.conv_out_hw(h, w, k, k, s, p)
    dy = rng.standard_normal((n, co, oh, ow)).astype(np.float32)
    _conv_check(g, x, wt, b, dy, s, p)


@pytest.mark.parametrize("cfg", [(8, 128, 16, 16, 128, 3, 1, 1, True), (3, 96, 20, 36, 72, 5, 1, 2, False), (4, 64, 56, 56, 64, 3, 1, 1, False)])
def test_conv_two_tiles_per_weight_stage(g, cfg, monkeypatch):
    """Large batches of layers with streamed weights compute two position tiles per weight stage; the
    batch threshold is lowered here so that small problems take that path too (odd tile counts, tiles
    straddling images, partial output-channel tiles)."""
    monkeypatch.setenv("MTB_ROWCONV_MIN_ITEMS", "1")
    n, ci, h, w, co, k, s, p, bias = cfg
    rng = np.random.default_rng(77)
    x = rng.standard_normal((n, ci, h, w)).astype(np.float32)
    wt = (rng.standard_normal((co, ci, k, k)) / np.sqrt(ci * k * k)).astype(np.float32)
    b = rng.standard_normal(co).astype(np.float32) if bias else None
    dy = rng.standard_normal((n, co, h, w)).astype(np.float32)
    _conv_check(g, x, wt, b, dy, s, p)


@pytest.mark.parametrize("cfg", [(8, 64, 32, 32, 64, 3, 1, 1), (8, 64, 32, 32, 128, 3, 2, 1), (2, 20, 9, 11, 24, 3, 1, 1), (8, 3, 32, 32, 64, 3, 1, 1),
                                 (8, 64, 32, 32, 128, 1, 2, 0), (16, 256, 8, 8, 512, 3, 2, 1), (64, 128, 16, 16, 256, 3, 2, 1)])
def test_conv_backward_accumulates_into_existing_gradient(g, cfg):
    """dx returned with ``accumulate_dx`` equals dgrad + that tensor bit for bit, on the row-staged
    path (sum in the epilogue), the im2col path (stride 2, also with residue classes side by side and classes
    without taps: sum afterwards), the CUDA-core path and the channel-padded stem."""
    n, ci, h, w, co, k, s, p = cfg
    rng = np.random.default_rng(11)
    x = rng.standard_normal((n, ci, h, w)).astype(np.float32)
    wt = rng.standard_normal((co, ci, k, k)).astype(np.float32)
    oh, ow = O.conv_out_hw(h, w, k, k, s, p)
    dy = rng.standard_normal((n, co, oh, ow)).astype(np.float32)
    prev = rng.standard_normal((n, ci, h, w)).astype(np.float32)
    xt, wtt, dyt, pt = g.dev(x, True), g.dev(wt, True), g.dev(dy), g.dev(prev)
    dx, _, _ = g.op("conv2d_backward")(dyt, xt, wtt, None, (s, s), (p, p))
    both, _, _ = g.op("conv2d_backward")(dyt, xt, wtt, None, (s, s), (p, p), accumulate_dx=pt)
    assert np.array_equal(g.host(both), g.host(dx) + prev)
    if k < s:  # a filter smaller than its stride accumulates in place: the tensor handed in is the one returned
        assert both is pt
    else:
        assert np.array_equal(g.host(pt), prev)


@pytest.mark.parametrize("shape", [(8, 64, 16, 16), (8, 256, 8, 8), (16, 512, 4, 4), (96, 64, 32, 32), (128, 128, 16, 16)])
def test_conv_is_deterministic(g, shape):
    """Bitwise-equal results on repeated runs, also for the layers whose forward pass and data gradient
    split their reduction across CTAs (few output tiles: 8x8 and 4x4 images), whose BatchNorm
    statistics come from the convolution's epilogue, and whose CTAs run several tiles issued by two
    warps in turn (the last two shapes: weights resident / streamed with two tiles per weight stage)."""
    n, c, h, w = shape
    rng = np.random.default_rng(5)
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = rng.standard_normal((c, c, 3, 3)).astype(np.float32)
    dy = rng.standard_normal((n, c, h, w)).astype(np.float32)
    gamma, beta = np.ones(c, np.float32), np.zeros(c, np.float32)
    outs = []
    for _ in range(3):
        xt, wtt = g.dev(x, True), g.dev(wt, True)
        y = g.op("conv2d")(xt, wtt, None, (1, 1), (1, 1), bn_stats=True)
        _, mean, var = g.op("batch_norm2d")(y, g.dev(gamma), g.dev(beta), 1e-5, True, 0.1, None, None)
        dx, dw, _ = g.op("conv2d_backward")(g.dev(dy), xt, wtt, None, (1, 1), (1, 1))
        outs.append((g.host(y), g.host(dx), g.host(dw), g.host(mean), g.host(var)))
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert np.array_equal(a, b)


def test_linear(g):
    gd = load_golden("misc")
    x, w, b, dy = g.dev(gd["lin_x"], True), g.dev(gd["lin_w"], True), g.dev(gd["lin_b"], True), g.dev(gd["lin_dy"])
    y = g.op("linear")(x, w, b)
    dx, dw, db = g.op("linear_backward")(dy, x, w, b)
    assert rel_err(g.host(y), gd["lin_y"]) < TF32_TOL and rel_err(g.host(dx), gd["lin_dx"]) < TF32_TOL
    assert rel_err(g.host(dw), gd["lin_dw"]) < TF32_TOL and rel_err(g.host(db), gd["lin_db"]) < FP32_TOL
    rng = np.random.default_rng(3)
    for (bsz, fin, fout) in [(64, 9216, 128), (64, 128, 10), (512, 512, 10), (128, 2048, 1000), (7, 33, 5)]:
        xa = rng.standard_normal((bsz, fin)).astype(np.float32)
        wa = (rng.standard_normal((fout, fin)) / np.sqrt(fin)).astype(np.float32)
        ba = rng.standard_normal(fout).astype(np.float32)
        da = rng.standard_normal((bsz, fout)).astype(np.float32)
        x, w, b = g.dev(xa, True), g.dev(wa, True), g.dev(ba, True)
        y = g.op("linear")(x, w, b)
        dx, dw, db = g.op("linear_backward")(g.dev(da), x, w, b)
        rdx, rdw, rdb = O.linear_backward(da, xa, wa, True)
        assert rel_err(g.host(y), O.linear_forward(xa, wa, ba)) < TF32_TOL
        assert rel_err(g.host(dx), rdx) < TF32_TOL and rel_err(g.host(dw), rdw) < TF32_TOL
        assert rel_err(g.host(db), rdb) < FP32_TOL * 10
        tx, tw, td = O.round_tf32(xa), O.round_tf32(wa), O.round_tf32(da)
        tdx, tdw, _ = O.linear_backward(td, tx, tw, False)
        assert _matches_a_model(g.host(y), O.linear_forward(xa, wa, ba), O.linear_forward(tx, tw, ba))
        assert _matches_a_model(g.host(dx), rdx, tdx) and _matches_a_model(g.host(dw), rdw, tdw)


def test_mm_and_permute(g):
    rng = np.random.default_rng(4)
    a, b = rng.standard_normal((37, 50)).astype(np.float32), rng.standard_normal((50, 21)).astype(np.float32)
    dy = rng.standard_normal((37, 21)).astype(np.float32)
    at, bt = g.dev(a, True), g.dev(b, True)
    assert rel_err(g.host(g.op("mm")(at, bt)), a @ b) < TF32_TOL
    da, db = g.op("mm_backward")(g.dev(dy), at, bt)
    assert rel_err(g.host(da), dy @ b.T) < TF32_TOL and rel_err(g.host(db), a.T @ dy) < TF32_TOL
    assert np.array_equal(g.host(g.op("permute")(at, (1, 0))), a.T)
    x4 = rng.standard_normal((2, 3, 4, 5)).astype(np.float32)
    assert np.array_equal(g.host(g.op("permute")(g.dev(x4), (0, 2, 3, 1))), x4.transpose(0, 2, 3, 1))
    assert np.array_equal(g.host(g.op("permute_backward")(g.dev(x4.transpose(2, 0, 3, 1).copy()), g.dev(x4), (2, 0, 3, 1))[0]), x4)


def test_layout_round_trip_and_reshape(g):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((3, 5, 4, 7)).astype(np.float32)
    xt = g.dev(x)
    assert np.array_equal(g.host(xt), x)
    flat = g.op("reshape")(xt, (3, -1))
    assert flat.shape == (3, 140) and np.array_equal(g.host(flat), x.reshape(3, -1))
    back = g.op("reshape")(flat, (3, 5, 4, 7))
    assert np.array_equal(g.host(back), x)
    assert np.array_equal(g.host(g.op("reshape")(g.dev(x[:, :, :1, :1].copy()), (3, 5))), x[:, :, 0, 0])


def test_batch_norm_golden_and_oracle(g):
    gd = load_golden("batch_norm")
    for i in range(int(gd["count"])):
        x, gm, b, rm, rv, dy = (gd[f"b{i}_{k}"] for k in ("x", "g", "b", "rm", "rv", "dy"))
        xt, gt, bt, rmt, rvt = g.dev(x, True), g.dev(gm, True), g.dev(b, True), g.dev(rm), g.dev(rv)
        y, mean, var = g.op("batch_norm2d")(xt, gt, bt, 1e-5, True, 0.1, rmt, rvt)
        assert rel_err(g.host(y), gd[f"b{i}_y"]) < FP32_TOL
        assert rel_err(g.host(rmt), gd[f"b{i}_rm2"]) < FP32_TOL and rel_err(g.host(rvt), gd[f"b{i}_rv2"]) < FP32_TOL
        dx, dg, db = g.op("batch_norm2d_backward")(g.dev(dy), mean, var, xt, gt, bt, 1e-5)
        assert rel_err(g.host(dx), gd[f"b{i}_dx"]) < FP32_TOL * 2
        assert rel_err(g.host(dg), gd[f"b{i}_dg"]) < FP32_TOL * 2 and rel_err(g.host(db), gd[f"b{i}_db"]) < FP32_TOL * 2
        ye, _, _ = g.op("batch_norm2d")(g.dev(x), g.dev(gm), g.dev(b), 1e-5, False, 0.1, g.dev(rm), g.dev(rv))
        assert rel_err(g.host(ye), gd[f"b{i}_yeval"]) < FP32_TOL
    rng = np.random.default_rng(7)
    for shp in [(16, 128, 28, 28), (32, 64, 32, 32), (8, 512, 4, 4), (5, 24, 9, 9), (4, 7, 6, 6)]:
        c = shp[1]
        x = (0.5 + 2.0 * rng.standard_normal(shp)).astype(np.float32)
        gm, b = rng.uniform(0.5, 1.5, c).astype(np.float32), rng.standard_normal(c).astype(np.float32)
        dy = rng.standard_normal(shp).astype(np.float32)
        ry, rmean, rvar, rrm, rrv = O.batch_norm2d_forward(x, gm, b, 1e-5, True, 0.1, np.zeros(c, np.float32), np.ones(c, np.float32))
        rdx, rdg, rdb = O.batch_norm2d_backward(dy, rmean, rvar, x, gm, 1e-5)
        xt, gt, bt, rmt, rvt = g.dev(x, True), g.dev(gm, True), g.dev(b, True), g.dev(np.zeros(c, np.float32)), g.dev(np.ones(c, np.float32))
        y, mean, var = g.op("batch_norm2d")(xt, gt, bt, 1e-5, True, 0.1, rmt, rvt)
        dx, dg, db = g.op("batch_norm2d_backward")(g.dev(dy), mean, var, xt, gt, bt, 1e-5)
        assert rel_err(g.host(y), ry) < FP32_TOL and rel_err(g.host(mean), rmean.reshape(-1)) < FP32_TOL
        assert rel_err(g.host(var), rvar.reshape(-1)) < FP32_TOL
        assert rel_err(g.host(rmt), rrm) < FP32_TOL and rel_err(g.host(rvt), rrv) < FP32_TOL
        assert rel_err(g.host(dx), rdx) < FP32_TOL * 2 and rel_err(g.host(dg), rdg) < FP32_TOL * 3 and rel_err(g.host(db), rdb) < FP32_TOL * 3


def test_max_pool_bit_exact(g):
    from mytorch_b200.backends.cuda.ops import max_pool2d_argmax

    gd = load_golden("max_pool")
    for i in range(int(gd["count"])):
        k, s, p, _ = (int(v) for v in gd[f"p{i}_cfg"])
        x, dy = gd[f"p{i}_x"], gd[f"p{i}_dy"]
        xt = g.dev(x, True)
        y = g.op("max_pool2d")(xt, (k, k), (s, s), (p, p))
        assert np.array_equal(g.host(y), gd[f"p{i}_y"])
        assert np.array_equal(max_pool2d_argmax(y), O.max_pool2d_argmax(x, k, s, p).astype(np.uint8))
        (dx,) = g.op("max_pool2d_backward")(g.dev(dy), y, xt, (k, k), (s, s), (p, p))
        assert rel_err(g.host(dx), gd[f"p{i}_dx"]) < 1e-6
        y._pool_tiemask = None  # force the x == out recomputation path
        (dx2,) = g.op("max_pool2d_backward")(g.dev(dy), y, xt, (k, k), (s, s), (p, p))
        assert np.array_equal(g.host(dx2), g.host(dx))
    rng = np.random.default_rng(8)
    for shp, k, s, p in [((8, 128, 56, 56), 2, 2, 0), ((4, 64, 112, 112), 3, 2, 1), ((2, 6, 9, 9), 5, 2, 2), ((3, 5, 7, 7), 2, 2, 0)]:
        x = rng.standard_normal(shp).astype(np.float32)
        xt = g.dev(x, True)
        y = g.op("max_pool2d")(xt, (k, k), (s, s), (p, p))
        ry = O.max_pool2d_forward(x, k, s, p)
        assert np.array_equal(g.host(y), ry)
        dy = rng.standard_normal(ry.shape).astype(np.float32)
        (dx,) = g.op("max_pool2d_backward")(g.dev(dy), y, xt, (k, k), (s, s), (p, p))
        assert rel_err(g.host(dx), O.max_pool2d_backward(dy, ry, x, k, s, p)) < 1e-6
        if k * k <= 16:
            assert np.array_equal(max_pool2d_argmax(y), O.max_pool2d_argmax(x, k, s, p).astype(np.uint8))


def test_elementwise_and_reductions(g):
    gd = load_golden("misc")
    assert np.array_equal(g.host(g.op("relu")(g.dev(gd["relu_x"]))), gd["relu_y"])
    assert np.array_equal(g.host(g.op("relu_backward")(g.dev(gd["relu_dy"]), g.dev(gd["relu_x"]))[0]), gd["relu_dx"])
    a, b = g.dev(gd["add_a"], True), g.dev(gd["add_b"], True)
    assert np.array_equal(g.host(g.op("add")(a, b, 1)), gd["add_y"])
    da, db = g.op("add_backward")(g.dev(gd["add_dy"]), a, b, 1)
    assert np.array_equal(g.host(da), gd["add_da"]) and np.array_equal(g.host(db), gd["add_db"])
    a, b = g.dev(gd["badd_a"], True), g.dev(gd["badd_b"], True)
    assert np.array_equal(g.host(g.op("add")(a, b, 1)), gd["badd_y"])
    da, db = g.op("add_backward")(g.dev(gd["badd_dy"]), a, b, 1)
    assert np.array_equal(g.host(da), gd["badd_da"]) and rel_err(g.host(db), gd["badd_db"]) < FP32_TOL
    x = g.dev(gd["gap_x"], True)
    assert rel_err(g.host(g.op("sum_scale")(x, (2, 3), False, 1 / 16)), gd["gap_y"]) < FP32_TOL
    assert rel_err(g.host(g.op("sum_scale_backward")(g.dev(gd["gap_dy"]), x, (2, 3), False, 1 / 16)[0]), gd["gap_dx"]) < FP32_TOL
    assert rel_err(g.host(g.op("sum_scale")(x, (0, 2, 3), False, 1)), gd["csum_y"]) < FP32_TOL
    assert rel_err(g.host(g.op("sum_scale_backward")(g.dev(gd["csum_dy"]), x, (0, 2, 3), False, 1)[0]), gd["csum_dx"]) < FP32_TOL
    xs = gd["gap_x"]
    for dim, keep in [((1,), False), ((0, 1, 2, 3), False), ((3,), True), ((0,), True), ((1, 2), False)]:
        r = O.sum_scale_forward(xs, dim, keep, 0.5)
        out = g.op("sum_scale")(x, dim, keep, 0.5)
        assert out.shape == r.shape and rel_err(g.host(out), r) < FP32_TOL
        dyv = np.random.default_rng(9).standard_normal(r.shape).astype(np.float32)
        dxv = g.op("sum_scale_backward")(g.dev(dyv), x, dim, keep, 0.5)[0]
        assert rel_err(g.host(dxv), O.sum_scale_backward(dyv, xs.shape, dim, keep, 0.5)) < FP32_TOL
    rng = np.random.default_rng(10)
    p, q = rng.standard_normal((4, 3, 5, 5)).astype(np.float32), rng.standard_normal((1, 3, 1, 1)).astype(np.float32)
    for name, f in [("add", lambda u, v: u + 2 * v), ("sub", lambda u, v: u - 2 * v)]:
        assert rel_err(g.host(g.op(name)(g.dev(p), g.dev(q), 2)), f(p, q)) < FP32_TOL
    assert rel_err(g.host(g.op("mul")(g.dev(p), g.dev(q))), p * q) < FP32_TOL
    assert rel_err(g.host(g.op("div")(g.dev(p), g.dev(np.abs(q) + 1))), p / (np.abs(q) + 1)) < FP32_TOL
    dp, dq = g.op("mul_backward")(g.dev(p), g.dev(p, True), g.dev(q, True))
    rp, rq = O.mul_backward(p, p, q)
    assert rel_err(g.host(dp), rp) < FP32_TOL and rel_err(g.host(dq), rq) < FP32_TOL


def test_cross_entropy(g):
    gd = load_golden("misc")
    z, t = g.dev(gd["ce_z"], True), g.dev(gd["ce_t"])
    loss = g.op("cross_entropy")(z, t)
    assert loss.shape == (1,) and rel_err(g.host(loss), gd["ce_loss"]) < FP32_TOL
    (dz,) = g.op("cross_entropy_backward")(g.dev(np.ones(1, np.float32)), z, t)
    assert rel_err(g.host(dz), gd["ce_dz"]) < FP32_TOL
    rng = np.random.default_rng(11)
    for b, c in [(512, 10), (128, 1000), (3, 37)]:
        za, ta = (4 * rng.standard_normal((b, c))).astype(np.float32), rng.integers(0, c, b).astype(np.int64)
        zt = g.dev(za, True)
        assert rel_err(g.host(g.op("cross_entropy")(zt, g.dev(ta))), O.cross_entropy_forward(za, ta)) < FP32_TOL
        (dz,) = g.op("cross_entropy_backward")(g.dev(np.full(1, 0.7, np.float32)), zt, g.dev(ta))
        assert rel_err(g.host(dz), O.cross_entropy_backward(np.float32(0.7), za, ta)) < FP32_TOL


def test_sgd(g):
    import mytorch_b200 as mt
    import mytorch_b200.nn as nn
    from mytorch_b200.optim import SGD

    gd = load_golden("misc")
    cfgs = [dict(lr=0.1, momentum=0.9), dict(lr=0.05, momentum=0.8, nesterov=True, weight_decay=1e-2),
            dict(lr=0.01, momentum=0.5, dampening=0.3, maximize=True)]
    for i, kw in enumerate(cfgs):
        for multi in (True, False):
            p = nn.Parameter(g.dev(gd[f"sgd{i}_p0"].copy()))
            opt = SGD([p], **kw)
            for gname, pname in (("g1", "p1"), ("g2", "p2")):
                p.grad = g.dev(gd[f"sgd{i}_{gname}"])
                if multi:
                    opt.step()
                else:
                    st = opt.state.setdefault(p, {})
                    first = "momentum_buffer" not in st
                    if first:
                        st["momentum_buffer"] = mt.Tensor(shape=p.shape, device=p.device, dtype=p.dtype)
                    g.op("sgd")(p, st["momentum_buffer"], first, kw["lr"], kw.get("weight_decay", 0), kw["momentum"],
                                kw.get("dampening", 0), kw.get("nesterov", False), kw.get("maximize", False))
                assert rel_err(g.host(p.detach()), gd[f"sgd{i}_{pname}"]) < FP32_TOL
            assert rel_err(g.host(opt.state[p]["momentum_buffer"]), gd[f"sgd{i}_buf"]) < FP32_TOL


def test_sgd_multi_tensor_over_ragged_sizes(g):
    """One multi-tensor launch over tensors of very different sizes (a CTA per 4096 elements of one tensor):
    sizes below, at and just past a chunk, an odd tail, and a second step that reads the momentum buffer."""
    import mytorch_b200.nn as nn
    from mytorch_b200.optim import SGD

    rng = np.random.default_rng(21)
    sizes = [1, 3, 64, 4095, 4096, 4097, 3 * 4096 + 5, 70001, 8]
    kw = dict(lr=0.05, momentum=0.9, weight_decay=1e-3, nesterov=True)
    host_p = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    host_b = [None] * len(sizes)
    params = [nn.Parameter(g.dev(a.copy())) for a in host_p]
    opt = SGD(params, **kw)
    for step in range(2):
        grads = [rng.standard_normal(n).astype(np.float32) for n in sizes]
        for p, gr in zip(params, grads):
            p.grad = g.dev(gr)
        opt.step()
        for i, gr in enumerate(grads):
            host_p[i], host_b[i] = O.sgd_step(host_p[i], gr, host_b[i], step == 0, **kw)
        for i, p in enumerate(params):
            assert rel_err(g.host(p.detach()), host_p[i]) < FP32_TOL, (step, sizes[i])
            assert rel_err(g.host(opt.state[p]["momentum_buffer"]), host_b[i]) < FP32_TOL, (step, sizes[i])


def test_strided_data_gradient_side_by_side_equals_serial(g, monkeypatch):
    """The residue classes of a strided data gradient run on separate lanes when each fills only part of the
    GPU; the result is bit-identical to running them one after the other."""
    rng = np.random.default_rng(8)
    for (n, cin, cout, hw, k, pad) in [(16, 64, 128, 32, 3, 1), (8, 128, 256, 16, 3, 1), (16, 64, 128, 32, 1, 0)]:
        x = rng.standard_normal((n, cin, hw, hw)).astype(np.float32)
        wt = (rng.standard_normal((cout, cin, k, k)) / 16).astype(np.float32)
        dy = rng.standard_normal((n, cout, hw // 2, hw // 2)).astype(np.float32)
        results = []
        for serial in (False, True):
            if serial:
                monkeypatch.setenv("MTB_DGRAD_SERIAL", "1")
            else:
                monkeypatch.delenv("MTB_DGRAD_SERIAL", raising=False)
            dx, _, _ = g.op("conv2d_backward")(g.dev(dy), g.dev(x, True), g.dev(wt, True), None, (2, 2), (pad, pad))
            results.append(g.host(dx))
        monkeypatch.delenv("MTB_DGRAD_SERIAL", raising=False)
        assert np.array_equal(results[0], results[1])
        ref = O.conv2d_backward(dy, x, wt, False, (2, 2), (pad, pad))[0]
        assert rel_err(results[0], ref) < TF32_TOL


def test_errors_are_python_exceptions(g):
    import mytorch_b200 as mt

    x = g.dev(np.zeros((1, 3, 8, 8), np.float32))
    w = g.dev(np.zeros((4, 5, 3, 3), np.float32))
    with pytest.raises(RuntimeError):
        g.op("conv2d")(x, w, None, (1, 1), (0, 0))
    with pytest.raises(RuntimeError):
        g.op("cross_entropy")(g.dev(np.zeros((2, 3), np.float32)), g.dev(np.zeros(2, np.int32)))
    with pytest.raises(RuntimeError):
        mt.tensor(np.zeros(3, np.int64), device="cuda:0", requires_grad=True)


def test_bounded_wait_runs_out_reports_once_and_leaves_the_context_usable(g):
    """The give-up path shared by all tensor-core kernels: a wait that nothing will ever satisfy
    ends after its limit, the status word carries the code exactly once, tensor memory is released
    (a convolution that needs all of it still runs) and results afterwards are bit-identical."""
    from mytorch_b200.backends.cuda.env import CudaEnv

    env = CudaEnv.instance()
    rng = np.random.default_rng(3)
    x = rng.standard_normal((8, 64, 32, 32)).astype(np.float32)
    w = rng.standard_normal((64, 64, 3, 3)).astype(np.float32)
    dy = rng.standard_normal((8, 64, 32, 32)).astype(np.float32)

    def conv():
        xt, wt = g.dev(x, True), g.dev(w, True)
        y = g.op("conv2d")(xt, wt, None, (1, 1), (1, 1))
        dx, dw, _ = g.op("conv2d_backward")(g.dev(dy), xt, wt, None, (1, 1), (1, 1))
        return g.host(y), g.host(dx), g.host(dw)

    before = conv()
    assert env.tensor_core_status() == 0
    env.lib.tc_wait_selftest(2_000_000, 77, env.stream())   # about one millisecond of SM cycles
    assert env.tensor_core_status() == 77
    assert env.tensor_core_status() == 0                     # reading cleared it
    after = conv()
    assert env.tensor_core_status() == 0
    for a, b in zip(before, after):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("cfg", [
    # n, cin, h, w, cout, k, s, p, bias        kernel the forward pass takes
    (8, 64, 32, 32, 64, 3, 1, 1, None),      # row-staged, resident filter
    (8, 64, 32, 32, 64, 3, 1, 1, 40.0),      # the same with a bias far larger than the spread of the outputs
    (16, 128, 16, 16, 128, 3, 1, 1, None),   # row-staged, streamed filter
    (3, 32, 17, 23, 96, 3, 1, 1, 1.0),       # row-staged, odd image, tiles straddling images
    (16, 256, 8, 8, 256, 3, 1, 1, None),     # im2col kernel
    (8, 64, 32, 32, 128, 3, 2, 1, None),     # im2col kernel, stride 2
    (32, 512, 4, 4, 512, 3, 1, 1, None),     # im2col kernel, several column tiles per row tile
    (8, 3, 32, 32, 64, 3, 1, 1, None),       # image stem (channels padded to one block)
    (8, 64, 32, 32, 128, 1, 2, 0, None),     # 1x1 shortcut, small output: statistics although the reduction is short
    (128, 64, 32, 32, 128, 1, 2, 0, None),   # 1x1 shortcut, 17 MB of output: too short a reduction, no statistics expected
])
def test_conv_epilogue_hands_batch_norm_its_statistics(g, cfg, monkeypatch):
    """A convolution asked for BatchNorm statistics leaves partial (count, mean, M2) rows on its output;
    BatchNorm forward from those rows matches the oracle's BatchNorm of that very output, and
    BatchNorm's own statistics pass, to fp32 accuracy.  The convolution's output itself is bit-identical
    with and without the statistics."""
    n, ci, h, w, co, k, s, p, bias = cfg
    if cfg[1] == 128:
        monkeypatch.setenv("MTB_ROWCONV_MIN_ITEMS", "1")   # two position tiles per weight stage
    rng = np.random.default_rng(abs(hash(cfg)) % (2 ** 31))
    x = rng.standard_normal((n, ci, h, w)).astype(np.float32)
    wt = (rng.standard_normal((co, ci, k, k)) / np.sqrt(ci * k * k)).astype(np.float32)
    b = None if bias is None else (bias + rng.standard_normal(co)).astype(np.float32)
    gamma, beta = rng.uniform(0.5, 1.5, co).astype(np.float32), rng.standard_normal(co).astype(np.float32)
    xt, wtt, bt = g.dev(x), g.dev(wt), (g.dev(b) if b is not None else None)
    plain = g.op("conv2d")(xt, wtt, bt, (s, s), (p, p))
    fused = g.op("conv2d")(xt, wtt, bt, (s, s), (p, p), bn_stats=True)
    yh = g.host(fused)
    assert np.array_equal(yh, g.host(plain))
    oh, ow = O.conv_out_hw(h, w, k, k, s, p)
    expect_stats = k > 1 or n * oh * ow * co * 4 <= (12 << 20)
    assert (getattr(fused, "_bn_partials", None) is not None) == expect_stats
    outs = []
    for src in (fused, plain):
        rm, rv = g.dev(np.zeros(co, np.float32)), g.dev(np.ones(co, np.float32))
        y, mean, var = g.op("batch_norm2d")(src, g.dev(gamma), g.dev(beta), 1e-5, True, 0.1, rm, rv)
        outs.append([g.host(t) for t in (y, mean, var, rm, rv)])
    ry, rmean, rvar, rrm, rrv = O.batch_norm2d_forward(yh, gamma, beta, 1e-5, True, 0.1, np.zeros(co, np.float32), np.ones(co, np.float32))
    for got in outs:
        assert rel_err(got[0], ry) < 2 * FP32_TOL
        assert rel_err(got[1], rmean.reshape(-1)) < FP32_TOL and rel_err(got[2], rvar.reshape(-1)) < 2 * FP32_TOL
        assert rel_err(got[3], rrm) < FP32_TOL and rel_err(got[4], rrv) < 2 * FP32_TOL
    assert rel_err(outs[0][1], outs[1][1]) < FP32_TOL and rel_err(outs[0][2], outs[1][2]) < 2 * FP32_TOL


def test_max_with_indices_and_its_backward(g):
    import mytorch_b200 as mt

    rng = np.random.default_rng(21)
    cases = [((7, 13), 1, False), ((7, 13), 0, True), ((3, 5, 6, 4), 1, False), ((3, 5, 6, 4), 3, True), ((3, 5, 6, 4), -2, False),
             ((4, 300), 1, False), ((2, 3, 4), None, False), ((3, 5, 6, 4), None, False)]
    for shape, dim, keep in cases:
        x = rng.integers(-4, 5, shape).astype(np.float32)   # many ties: the first maximum must win
        xt = g.dev(x, True)
        out = mt.max(xt, dim, keep)
        rv, ri = O.max_forward(x, dim, keep)
        if dim is None:
            values = out
            assert np.array_equal(g.host(values.detach()), rv)
        else:
            values, indices = out
            assert np.array_equal(g.host(values.detach()), rv) and np.array_equal(g.host(indices), ri)
        dy = rng.standard_normal(rv.shape if rv.shape else (1,)).astype(np.float32).reshape(rv.shape)
        node = values._grad_node
        (dx,) = g.op("max_backward")(g.dev(dy), node.helpers[0], xt, dim, keep)
        assert np.array_equal(g.host(dx), O.max_backward(dy, O.max_forward(x, dim, keep)[1], x.shape, dim, keep))


def test_eq_bmm_and_the_remaining_binary_gradients(g):
    import mytorch_b200 as mt

    rng = np.random.default_rng(22)
    for shape in [(5, 7), (2, 3, 4, 5)]:
        a = rng.integers(0, 3, shape).astype(np.float32)
        b = rng.integers(0, 3, shape).astype(np.float32)
        assert np.array_equal(g.host(g.dev(a).eq(g.dev(b))), O.eq_forward(a, b))
    ia, ib = rng.integers(0, 4, (33,)).astype(np.int64), rng.integers(0, 4, (33,)).astype(np.int64)
    assert np.array_equal(g.host(mt.eq(g.dev(ia), g.dev(ib))), O.eq_forward(ia, ib))
    # batched product: a CUDA-core sized case and a tensor-core sized one
    for bsz, m, k, n in [(3, 5, 7, 6), (2, 64, 96, 48)]:
        x = rng.standard_normal((bsz, m, k)).astype(np.float32)
        y = rng.standard_normal((bsz, k, n)).astype(np.float32)
        dz = rng.standard_normal((bsz, m, n)).astype(np.float32)
        xt, yt = g.dev(x, True), g.dev(y, True)
        assert rel_err(g.host(mt.bmm(xt, yt).detach()), O.bmm_forward(x, y)) < TF32_TOL
        dx, dy = g.op("bmm_backward")(g.dev(dz), xt, yt)
        rdx, rdy = O.bmm_backward(dz, x, y)
        assert rel_err(g.host(dx), rdx) < TF32_TOL and rel_err(g.host(dy), rdy) < TF32_TOL
    # div / pow gradients, same shape and broadcast
    for xs, ys in [((4, 6), (4, 6)), ((4, 6), (6,)), ((2, 3, 4, 5), (1, 3, 1, 1))]:
        x = rng.uniform(0.5, 2.0, xs).astype(np.float32)
        y = rng.uniform(0.5, 2.0, ys).astype(np.float32)
        dz = rng.standard_normal(np.broadcast_shapes(xs, ys)).astype(np.float32)
        for name, ref in (("div_backward", O.div_backward), ("pow_backward", O.pow_backward)):
            gx, gy = g.op(name)(g.dev(dz), g.dev(x), g.dev(y))
            rx, ry = ref(dz, x, y)
            assert rel_err(g.host(gx), rx) < 2 * FP32_TOL and rel_err(g.host(gy), ry) < 2 * FP32_TOL, (name, xs, ys)
    # through the tape
    x, y = g.dev(rng.uniform(0.5, 2.0, (3, 4)).astype(np.float32), True), g.dev(rng.uniform(0.5, 2.0, (4,)).astype(np.float32), True)
    ((x / y) ** y).sum().backward()
    assert x.grad.shape == (3, 4) and y.grad.shape == (4,)


def test_batch_norm_1d(g):
    import mytorch_b200.nn as nn

    rng = np.random.default_rng(23)
    for shape in [(16, 12), (6, 12, 10)]:
        x = (1.0 + rng.standard_normal(shape)).astype(np.float32)
        dy = rng.standard_normal(shape).astype(np.float32)
        bn = nn.BatchNorm1d(12)
        bn.to(g.DEV)
        xt = g.dev(x, True)
        y = bn(xt)
        (y * g.dev(dy)).sum().backward()
        x4 = x.reshape(shape[0], 12, -1, 1)
        ry, mean, var, rm, rv = O.batch_norm2d_forward(x4, np.ones(12, np.float32), np.zeros(12, np.float32), 1e-5, True, 0.1,
                                                        np.zeros(12, np.float32), np.ones(12, np.float32))
        rdx, rdg, rdb = O.batch_norm2d_backward(dy.reshape(x4.shape), mean, var, x4, np.ones(12, np.float32), 1e-5)
        assert rel_err(g.host(y.detach()), ry.reshape(shape)) < FP32_TOL
        assert rel_err(g.host(xt.grad), rdx.reshape(shape)) < 2 * FP32_TOL
        assert rel_err(g.host(bn.weight.grad), rdg) < 3 * FP32_TOL and rel_err(g.host(bn.bias.grad), rdb) < 3 * FP32_TOL
        assert rel_err(g.host(bn.running_mean), rm) < FP32_TOL and rel_err(g.host(bn.running_var), rv) < FP32_TOL
