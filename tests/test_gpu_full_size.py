"""Parity at the sizes the benchmark times.

Kernel selection depends on the problem size (two position tiles per weight stage above a work
threshold, tile widths narrowed for small problems, split counts), so the shapes `bench.py` runs
are checked here at their full size:

* configs[1]: Conv2d 64->64 3x3 s1 p1 + bias on 128x64x56x56, forward, dgrad, wgrad, bias gradient,
  against the oracle (5e-3 for the TF32 results, 1e-5 for the fp32 bias gradient);
* configs[2]: BatchNorm2d(128) -> ReLU -> MaxPool2d(2,2) on 256x128x56x56, forward and backward,
  against the oracle (1e-5-class), pooled values and argmax bit-exact on the pooling input the GPU
  itself produced;
* configs[3]: one ResNet-18 step at the global batch of 512 against gradients recorded from the
  reference's own CPU backend (tests/golden/data_parallel.npz, 64 samples and the norm of every
  parameter gradient), and at batch 128 against the oracle with every gradient element.

Whole-step bounds.  The first loss is held to 5e-3 (measured: 6e-5).  The gradient of this
network at its initial weights is ill-conditioned: the oracle run in float64 and the oracle run in
float32 differ by 5e-3 in relative L2 over the whole gradient vector (amplification ~1e5 of fp32
rounding), and the oracle with nothing changed but its GEMM operands rounded to TF32 (exact
accumulation) differs from itself by 9e-2 (tests/test_oracle_conditioning.py reproduces both on the
CPU).  The GPU measures the same: 9.2e-2 on the TF32 tensor-core kernels, 8e-3 on the fp32 CUDA-core
kernels, both against the oracle at batch 128.  End-to-end gradients are therefore held to
GRAD_L2 = 0.15 (1.6 x measured) for TF32 and GRAD_L2_FP32 = 2.5e-2 (3 x measured) for the fp32
kernels; the 5e-3 bound is enforced where it is well-posed, operator by operator on identical
inputs (tests/layerwise.py, used by tests/test_gpu_models.py).
"""
import numpy as np
import pytest

from conftest import load_golden, rel_err, rel_l2, summarize
from oracle import models as OM
from oracle import ops as O

pytestmark = pytest.mark.gpu

TF32_TOL = 5e-3
FP32_TOL = 1e-5
LOSS_TOL = 5e-3
GRAD_L2 = 0.15          # whole gradient vector, relative L2, TF32 path (measured 0.092)
GRAD_L2_TENSOR = 0.30   # any single parameter's gradient, relative L2 (measured 0.125)
GRAD_L2_FP32 = 2.5e-2   # the same step on the fp32 CUDA-core kernels (measured 0.0081)


def test_config1_conv_full_size_matches_oracle():
    import gpu_util as g

    rng = np.random.default_rng(1001)
    n, c, hw = 128, 64, 56
    x = rng.standard_normal((n, c, hw, hw)).astype(np.float32)
    dy = rng.standard_normal((n, c, hw, hw)).astype(np.float32)
    bound = 1.0 / np.sqrt(c * 9)
    w = rng.uniform(-bound, bound, (c, c, 3, 3)).astype(np.float32)
    b = rng.uniform(-bound, bound, c).astype(np.float32)
    xt, wt, bt = g.dev(x, True), g.dev(w, True), g.dev(b, True)
    y = g.op("conv2d")(xt, wt, bt, (1, 1), (1, 1))
    dx, dw, db = g.op("conv2d_backward")(g.dev(dy), xt, wt, bt, (1, 1), (1, 1))
    y, dx, dw, db = g.host(y), g.host(dx), g.host(dw), g.host(db)
    ry = O.conv2d_forward(x, w, b, (1, 1), (1, 1))
    assert rel_err(y, ry) < TF32_TOL
    del ry
    rdx, rdw, rdb = O.conv2d_backward(dy, x, w, True, (1, 1), (1, 1))
    assert rel_err(dx, rdx) < TF32_TOL
    assert rel_err(dw, rdw) < TF32_TOL
    # 401,408 signed terms per channel: the sum is ~270 times smaller than the sum of magnitudes, and
    # the quotient below is relative to the largest sum, so fp32 summation (either side) shows at 1e-5
    assert rel_err(db, dy.astype(np.float64).sum(axis=(0, 2, 3))) < 3 * FP32_TOL


def test_config2_bn_relu_pool_full_size_matches_oracle():
    import gpu_util as g
    from mytorch_b200.backends.cuda.ops import max_pool2d_argmax

    rng = np.random.default_rng(1002)
    n, c, hw = 256, 128, 56
    x = (0.5 + 2.0 * rng.standard_normal((n, c, hw, hw), dtype=np.float32)).astype(np.float32)
    dy = rng.standard_normal((n, c, hw // 2, hw // 2), dtype=np.float32)
    gamma, beta = g.dev(np.ones(c, np.float32), True), g.dev(np.zeros(c, np.float32), True)
    rm, rv = g.dev(np.zeros(c, np.float32)), g.dev(np.ones(c, np.float32))
    xt = g.dev(x, True)
    bn, mean, var = g.op("batch_norm2d")(xt, gamma, beta, 1e-5, True, 0.1, rm, rv)
    act = g.op("relu")(bn)
    pooled = g.op("max_pool2d")(act, (2, 2), (2, 2), (0, 0))
    d_act, = g.op("max_pool2d_backward")(g.dev(dy), pooled, act, (2, 2), (2, 2), (0, 0))
    d_bn, = g.op("relu_backward")(d_act, bn)
    dx, dgamma, dbeta = g.op("batch_norm2d_backward")(d_bn, mean, var, xt, gamma, beta, 1e-5)

    # pooling on the very input the GPU pooled: values and argmax bit-exact
    act_h, pooled_h = g.host(act), g.host(pooled)
    assert np.array_equal(pooled_h, O.max_pool2d_forward(act_h, (2, 2), (2, 2), (0, 0)))
    assert np.array_equal(max_pool2d_argmax(pooled), O.max_pool2d_argmax(act_h, (2, 2), (2, 2), (0, 0)).astype(np.uint8))
    assert np.array_equal(g.host(d_act), O.max_pool2d_backward(dy, pooled_h, act_h, (2, 2), (2, 2), (0, 0)))
    del act_h

    # the whole block against the oracle
    ref = OM.bn_relu_pool_block(x, dy, c)
    assert rel_err(pooled_h, ref["y"]) < FP32_TOL
    assert rel_err(g.host(mean), ref["mean"]) < FP32_TOL and rel_err(g.host(var), ref["var"]) < FP32_TOL
    assert rel_err(g.host(rm), ref["running_mean"]) < FP32_TOL and rel_err(g.host(rv), ref["running_var"]) < FP32_TOL
    assert rel_err(g.host(dx), ref["dx"]) < 2 * FP32_TOL
    assert rel_err(g.host(dgamma), ref["dgamma"]) < 3 * FP32_TOL and rel_err(g.host(dbeta), ref["dbeta"]) < 3 * FP32_TOL


def _resnet_step(x, t, seed):
    import gpu_util as g
    import mytorch_b200 as mt
    import mytorch_b200.nn.functional as F
    from mytorch_b200.examples.models import ResNet18Cifar

    mt.manual_seed(seed)
    net = ResNet18Cifar()
    net.to(g.DEV)
    loss = F.cross_entropy(net(g.dev(x)), g.dev(t))
    loss.backward()
    return loss.item(), {k: g.host(v.grad).astype(np.float64) for k, v in net.named_parameters()}


def _grad_errors(got, ref):
    num = den = 0.0
    worst = 0.0
    for k, r in ref.items():
        r = np.asarray(r, np.float64)
        worst = max(worst, rel_l2(got[k], r))
        num += float(np.sum((got[k] - r) ** 2))
        den += float(np.sum(r ** 2))
    return (num / den) ** 0.5, worst


def _config3_batch():
    rng = np.random.default_rng(1003)
    x = rng.standard_normal((512, 3, 32, 32)).astype(np.float32)
    t = rng.integers(0, 10, 512).astype(np.int64)
    return x, t


def test_config3_resnet18_step_at_batch_512_matches_reference_fixture():
    gd = load_golden("data_parallel")
    x, t = _config3_batch()
    loss, grads = _resnet_step(x, t, 1003)
    ref_loss = float(gd["c3_b512/w1/loss"])
    assert abs(loss - ref_loss) < LOSS_TOL * abs(ref_loss), (loss, ref_loss)
    got = {k: summarize(v)[1] for k, v in grads.items()}
    ref = {k: gd[f"c3_b512/w1/grad/{k}/sample"] for k in grads}
    total, worst = _grad_errors(got, ref)
    assert total < GRAD_L2 and worst < GRAD_L2_TENSOR, (total, worst)
    for k, v in grads.items():  # norms of the full tensors
        rn = gd[f"c3_b512/w1/grad/{k}/stats"][2]
        assert abs(np.linalg.norm(v) - rn) < GRAD_L2_TENSOR * rn, k


def test_config3_resnet18_step_at_batch_128_matches_oracle_on_both_kernel_families(monkeypatch):
    x, t = _config3_batch()
    x, t = x[:128], t[:128]
    ref_net = OM.resnet18_cifar(1003)
    ref_loss, ref_grads, _ = ref_net.loss_and_grads(x, t)
    loss, grads = _resnet_step(x, t, 1003)
    assert abs(loss - ref_loss) < LOSS_TOL * abs(ref_loss), (loss, ref_loss)
    total, worst = _grad_errors(grads, ref_grads)
    assert total < GRAD_L2 and worst < GRAD_L2_TENSOR, (total, worst)
    # the same step on the fp32 CUDA-core kernels: no TF32 rounding, so the error drops to fp32 level
    monkeypatch.setenv("MTB_DISABLE_TC", "1")
    loss32, grads32 = _resnet_step(x, t, 1003)
    assert abs(loss32 - ref_loss) < 2e-5 * abs(ref_loss), (loss32, ref_loss)
    total32, _ = _grad_errors(grads32, ref_grads)
    assert total32 < GRAD_L2_FP32, total32
