"""Host-side behaviour that needs no GPU: tensor / device / module / optimizer semantics of the
reference API, seeded initialisation, and the C-ABI library's exported symbols."""
import ctypes
import os
import re

import numpy as np
import pytest

import mytorch_b200 as mt
import mytorch_b200.nn as nn
from conftest import ROOT, load_golden
from mytorch_b200.optim import SGD
from mytorch_b200.tensor import Device


def test_device_parsing_and_equality():
    assert Device("cuda:1").type == "cuda" and Device("cuda:1").index == 1
    assert Device(" cpu ").index is None and repr(Device("cuda:0")) == "cuda:0"
    assert Device("cuda:0") == Device(Device("cuda:0")) and Device("cuda") != Device("cuda:0")


def test_tensor_constructor_rules():
    t = mt.tensor([[1, 2], [3, 4]], dtype=mt.float32)
    assert t.shape == (2, 2) and t.dtype is mt.float32 and t.device == Device("cpu")
    assert mt.Tensor(shape=(2, 3), dtype=mt.int64)._numpy().sum() == 0
    with pytest.raises(RuntimeError):
        mt.tensor([1, 2], dtype=mt.int64, requires_grad=True)
    with pytest.raises(RuntimeError):
        mt.Tensor(cpu_array=np.zeros(3, np.float32), dtype=mt.float64)
    with pytest.raises(RuntimeError):
        mt.Tensor(cpu_array=np.zeros(3, np.float32), shape=(4,))
    g = mt.tensor([1.0], dtype=mt.float32, requires_grad=True)
    with pytest.raises(RuntimeError):
        g.numpy()
    assert g.detach().numpy()[0] == 1.0 and g.item() == 1.0
    assert "tensor(" in repr(g)


def test_no_cpu_compute_backend():
    x = mt.tensor(np.zeros((1, 1, 4, 4), np.float32))
    conv = nn.Conv2d(1, 2, 3)
    with pytest.raises(RuntimeError, match="no function registered for conv2d on cpu"):
        conv(x)


def test_seeded_init_matches_reference_fixture():
    g = load_golden("misc")
    mt.manual_seed(77)
    c, l = nn.Conv2d(3, 4, 3), nn.Linear(6, 5)
    assert np.array_equal(c.weight._numpy(), g["init_cw"]) and np.array_equal(c.bias._numpy(), g["init_cb"])
    assert np.array_equal(l.weight._numpy(), g["init_lw"]) and np.array_equal(l.bias._numpy(), g["init_lb"])


def test_module_registration_and_state_dict(tmp_path):
    from mytorch_b200.examples.models import ResNet18Cifar

    mt.manual_seed(1)
    net = ResNet18Cifar(widths=(4, 8, 8, 8))
    keys = list(net.state_dict().keys())
    assert keys[:6] == ["conv1.weight", "bn1.weight", "bn1.bias", "bn1.running_mean", "bn1.running_var",
                        "layer1.0.conv1.weight"]
    assert "layer2.0.downsample.0.weight" in keys and keys[-2:] == ["fc.weight", "fc.bias"]
    assert len(list(net.parameters())) == 62
    assert net.training and not net.eval().training and all(not m.training for _, m in net.named_modules())
    path = os.path.join(tmp_path, "ckpt.bin")
    mt.save(net.state_dict(), path)
    mt.manual_seed(2)
    other = ResNet18Cifar(widths=(4, 8, 8, 8))
    assert not np.array_equal(other.fc.weight._numpy(), net.fc.weight._numpy())
    other.load_state_dict(mt.load(path))
    for (k1, a), (k2, b) in zip(net.state_dict().items(), other.state_dict().items()):
        assert k1 == k2 and np.array_equal(a._numpy(), b._numpy())


def test_optimizer_groups_and_state():
    p, q = nn.Parameter(mt.tensor(np.ones(3, np.float32))), nn.Parameter(mt.tensor(np.ones(2, np.float32)))
    opt = SGD([{"params": [p], "lr": 0.5}, {"params": [q]}], lr=0.1, momentum=0.9)
    assert opt.param_groups[0]["lr"] == 0.5 and opt.param_groups[1]["lr"] == 0.1 and opt.param_groups[1]["momentum"] == 0.9
    with pytest.raises(RuntimeError):
        SGD([{"params": [p]}, {"params": [p]}])
    p.grad = mt.tensor(np.ones(3, np.float32))
    opt.zero_grad()
    assert p.grad is None
    sd = opt.state_dict()
    assert sd["param_groups"][0]["params"] == [id(p)]


def test_backward_requires_graph_and_scalar():
    t = mt.tensor([1.0, 2.0], dtype=mt.float32, requires_grad=True)
    with pytest.raises(RuntimeError, match="backward a tensor twice"):
        t.backward()
    with mt.no_grad():
        with mt.no_grad():
            pass
        from mytorch_b200.autograd import DAGTracker

        assert DAGTracker.instance().no_grad
    assert not DAGTracker.instance().no_grad


def test_tape_hands_accumulated_gradient_to_operators_that_can_add_it():
    """An operator listed in ``fused_accumulate`` receives the gradient its input already holds and
    returns the sum; the tape stores that instead of adding.  Leaves receive their last gradient
    exactly once through the hook, whatever the number of consumers."""
    from mytorch_b200.autograd import DAGTracker
    from mytorch_b200.ops._common import record

    tr = DAGTracker.instance()
    seen = []

    def scale_op(name, x, k):
        out = mt.tensor(x._numpy() * np.float32(k))
        out.requires_grad = True
        return record(name, [x, k], out)

    def total(x):  # a one-element tensor to call backward on
        out = mt.tensor(np.array([x._numpy().sum()], np.float32))
        out.requires_grad = True
        return record("t_sum", [x], out)

    @tr.register_backward_function("t_sum")
    def _(dy, x):
        return [mt.tensor(np.full(x.shape, dy._numpy()[0], np.float32))]

    @tr.register_backward_function("t_plain")
    def _(dy, x, k):
        return [mt.tensor(dy._numpy() * np.float32(k)), None]

    @tr.register_backward_function("t_fused")
    def _(dy, x, k, accumulate_dx=None):
        seen.append(None if accumulate_dx is None else accumulate_dx._numpy().copy())
        g = dy._numpy() * np.float32(k)
        return [mt.tensor(g if accumulate_dx is None else g + accumulate_dx._numpy()), None]

    @tr.register_backward_function("t_add")
    def _(dy, a, b):
        return [dy, dy]

    tr.fused_accumulate["t_fused"] = 0
    finals = []
    tr.leaf_grad_final_hook = lambda t: finals.append(id(t))
    try:
        x = mt.tensor(np.arange(4, dtype=np.float32), requires_grad=True)
        a = scale_op("t_fused", x, 2.0)      # created first, so its backward runs last
        b = scale_op("t_plain", x, 3.0)
        s = mt.tensor(a._numpy() + b._numpy())
        s.requires_grad = True
        record("t_add", [a, b], s)
        total(s).backward()
    finally:
        tr.leaf_grad_final_hook = None
        del tr.fused_accumulate["t_fused"]
    assert len(seen) == 1 and np.array_equal(seen[0], np.full(4, 3.0, np.float32))   # got the gradient from t_plain
    assert np.array_equal(x.grad._numpy(), np.full(4, 5.0, np.float32))
    assert finals == [id(x)]


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "mytorch_b200.h")).read()
    return sorted(set(re.findall(r"\b(mtb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from mytorch_b200.backends.cuda.env import LIBRARY_PATH, _SIGNATURES

    if not os.path.exists(LIBRARY_PATH):
        from mytorch_b200.build import build_library

        build_library()
    dll = ctypes.CDLL(LIBRARY_PATH)
    names = _declared_symbols()
    assert len(names) >= 35
    for name in names:
        assert hasattr(dll, name), f"{name} is declared in include/mytorch_b200.h but not exported"
    for name in _SIGNATURES:
        assert name in names, f"{name} is bound by the Python layer but not declared in the header"
    dll.mtb_version.restype = ctypes.c_int
    assert dll.mtb_version() >= 1


def test_row_staged_kernels_never_plan_to_leave_their_memory():
    """For every shape the row-staged tcgen05 kernels accept, the furthest byte their copies write and
    their shifted descriptors read lies inside the stage or panel it belongs to, the stages fit the
    227 KB of shared memory of a CTA and the accumulators fit the 512 columns of tensor memory.
    (Host-side planning code only: runs without a GPU.)"""
    from mytorch_b200.backends.cuda.env import LIBRARY_PATH

    lib = ctypes.CDLL(LIBRARY_PATH)
    lib.mtb_conv2d_plan_f32.argtypes = [ctypes.c_int] * 11 + [ctypes.POINTER(ctypes.c_int)]
    out = (ctypes.c_int * 25)()
    limit = 227 * 1024
    seen = {0: 0, 1: 0, 2: 0}
    sizes = [1, 2, 3, 4, 5, 7, 8, 9, 12, 14, 16, 17, 23, 28, 31, 32, 33, 40, 56, 57, 64, 100, 112, 127, 224, 250, 254, 255, 300]
    for k in (3, 5, 7, 9):
        p_ = k // 2
        for h in sizes:
            for w in sizes:
                for cin in (32, 64, 96, 160, 256, 512):
                    for cout in (4, 32, 64, 72, 128, 192, 256, 512):
                        for n in (1, 7, 512):
                            assert lib.mtb_conv2d_plan_f32(n, cin, h, w, k, k, 1, 1, p_, p_, cout, out) == 0
                            fwd, dgrad, wgrad = out[0], out[1], out[2]
                            seen[fwd] += 1
                            for path, o in ((fwd, 3), (dgrad, 10)):
                                if path == 2:
                                    smem, stage, written, read, tmem, mt, resident = (out[o + i] for i in range(7))
                                    assert 0 < smem <= limit and written <= stage and read <= stage, (n, cin, h, w, k, cout, list(out))
                                    assert tmem <= 512 and mt in (1, 2) and resident in (0, 1)
                            if wgrad == 2:
                                smem, xp, xw, xr, yp, yw, yr, tmem = (out[17 + i] for i in range(8))
                                assert 0 < smem <= limit and xw <= xp and xr <= xp and yw <= yp and yr <= yp, (n, cin, h, w, k, cout, list(out))
                                assert 0 < tmem <= 512
    for kh, kw in ((1, 3), (3, 1), (5, 3), (3, 7), (1, 9), (15, 3)):   # non-square filters
        for h in (8, 17, 32, 56):
            for w in (8, 17, 32, 56, 250):
                for cin, cout in ((32, 16), (64, 64), (128, 256)):
                    assert lib.mtb_conv2d_plan_f32(64, cin, h, w, kh, kw, 1, 1, kh // 2, kw // 2, cout, out) == 0
                    for path, o in ((out[0], 3), (out[1], 10)):
                        if path == 2:
                            assert 0 < out[o] <= limit and out[o + 2] <= out[o + 1] and out[o + 3] <= out[o + 1] and out[o + 4] <= 512, (kh, kw, h, w, list(out))
                    if out[2] == 2:
                        assert 0 < out[17] <= limit and out[19] <= out[18] and out[20] <= out[18] and out[22] <= out[21] and out[23] <= out[21] and out[24] <= 512
    assert seen[2] > 1000 and seen[1] > 1000   # the sweep reaches both tensor-core families
    # shapes of the ResNet-18 step: row-staged at 32x32 and 16x16, im2col-mode at 8x8 and 4x4, CUDA cores for tiny inputs
    for cfg, want in (((512, 64, 32, 32, 3, 3, 1, 1, 1, 1, 64), [2, 2, 2]), ((512, 128, 16, 16, 3, 3, 1, 1, 1, 1, 128), [2, 2, 2]),
                      ((512, 256, 8, 8, 3, 3, 1, 1, 1, 1, 256), [1, 1, 1]), ((512, 64, 32, 32, 3, 3, 2, 2, 1, 1, 128), [1, 1, 1]),
                      ((2, 20, 9, 11, 3, 3, 1, 1, 1, 1, 24), [0, 0, 0])):
        lib.mtb_conv2d_plan_f32(*cfg, out)
        assert list(out[0:3]) == want, (cfg, list(out))


def test_in_place_data_gradient_is_offered_only_where_the_filter_misses_pixels():
    """Host-side query: a strided convolution whose filter is smaller than the stride (the 1x1 / stride-2 shortcut)
    may add its data gradient in place; every other shape keeps the out-of-place form."""
    import ctypes

    from mytorch_b200.backends.cuda.env import LIBRARY_PATH

    lib = ctypes.CDLL(LIBRARY_PATH)
    fn = lib.mtb_conv2d_dgrad_accumulates_in_place
    fn.argtypes = [ctypes.c_int] * 11 + [ctypes.c_void_p] * 3
    fn.restype = ctypes.c_int
    aligned = (ctypes.c_void_p(1 << 20),) * 3  # never dereferenced: the query looks at alignment only
    assert fn(64, 64, 32, 32, 1, 1, 2, 2, 0, 0, 128, *aligned) == 1
    assert fn(64, 64, 32, 32, 3, 3, 2, 2, 1, 1, 128, *aligned) == 0  # every residue class has a tap
    assert fn(64, 64, 32, 32, 3, 3, 1, 1, 1, 1, 64, *aligned) == 0   # stride 1: summed in the epilogue, out of place
    assert fn(64, 64, 32, 32, 1, 1, 2, 2, 0, 0, 128, ctypes.c_void_p((1 << 20) + 4), *aligned[:2]) == 0  # unaligned
    assert fn(1, 3, 8, 8, 1, 1, 2, 2, 0, 0, 8, *aligned) == 0  # shapes the tensor-core family does not take


def test_shard_bounds_cover_batch():
    from mytorch_b200.parallel import shard_bounds

    for n in (512, 10, 7):
        for world in (1, 2, 4, 8):
            spans = [shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
