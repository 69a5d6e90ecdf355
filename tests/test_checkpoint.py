"""A checkpoint written by the reference's own ``mytorch.save`` (tests/golden/reference_checkpoint.pt, made
by tests/golden/make_golden.py) loads into this implementation: tensors, state-dict keys, optimizer
state.  On the GPU the loaded model and optimizer take the next SGD-momentum step and land where
the reference landed (the momentum buffers are therefore really in use), and a checkpoint saved
from the GPU round-trips through ``save`` / ``load``."""
import os

import numpy as np
import pytest

from conftest import GOLDEN, load_golden, rel_err

CKPT = os.path.join(GOLDEN, "reference_checkpoint.pt")


def _net(device="cpu"):
    import mytorch_b200.nn as nn
    from mytorch_b200.examples.models import Flatten

    return nn.Sequential(nn.Conv2d(3, 8, 3, 1, 1, device=device), nn.BatchNorm2d(8, device=device), nn.ReLU(), nn.MaxPool2d(2, 2), Flatten(),
                         nn.Linear(8 * 6 * 6, 5, device=device))


def _batch():
    rng = np.random.default_rng(3003)
    return rng.standard_normal((8, 3, 12, 12)).astype(np.float32), rng.integers(0, 5, 8).astype(np.int64)


def test_reference_checkpoint_loads_on_the_cpu():
    import mytorch_b200 as mt
    from mytorch_b200.optim import SGD

    gd = load_golden("checkpoint")
    ck = mt.load(CKPT)
    assert list(ck["model"].keys()) == ["0.weight", "0.bias", "1.weight", "1.bias", "1.running_mean", "1.running_var", "5.weight", "5.bias"]
    for k, v in ck["model"].items():
        assert v.device.type == "cpu" and np.array_equal(v._numpy(), gd[f"saved/{k}"])
    net = _net()
    net.load_state_dict(ck["model"])
    for k, v in net.state_dict().items():
        assert np.array_equal(v._numpy(), gd[f"saved/{k}"])
    opt = SGD(net.parameters(), lr=0.5)
    opt.load_state_dict(ck["optimizer"])
    for i, p in enumerate(net.parameters()):
        assert np.array_equal(opt.state[p]["momentum_buffer"]._numpy(), gd[f"momentum/{i}"])


@pytest.mark.gpu
def test_reference_checkpoint_continues_training_on_the_gpu(tmp_path):
    import gpu_util as g
    import mytorch_b200 as mt
    import mytorch_b200.nn.functional as F
    from mytorch_b200.optim import SGD

    gd = load_golden("checkpoint")
    ck = mt.load(CKPT, map_location=g.DEV)
    assert all(v.device.type == "cuda" for v in ck["model"].values())
    net = _net()
    net.to(g.DEV)
    net.load_state_dict(ck["model"])
    opt = SGD(net.parameters(), lr=0.05, momentum=0.9)
    opt.load_state_dict(ck["optimizer"])
    x, t = _batch()
    loss = F.cross_entropy(net(g.dev(x)), g.dev(t))
    opt.zero_grad()
    loss.backward()
    opt.step()
    assert abs(loss.item() - float(gd["loss1"])) < 5e-3 * abs(float(gd["loss1"]))
    for k, v in net.state_dict().items():
        assert rel_err(g.host(v), gd[f"next/{k}"]) < 5e-3, k
    # and back: a checkpoint saved from GPU tensors holds logical-layout arrays and reloads bit for bit
    path = str(tmp_path / "roundtrip.pt")
    mt.save({"model": net.state_dict(), "optimizer": opt.state_dict()}, path)
    again = mt.load(path, map_location="cpu")
    for k, v in net.state_dict().items():
        assert np.array_equal(again["model"][k]._numpy(), g.host(v))
    net2 = _net()
    net2.to(g.DEV)
    net2.load_state_dict(mt.load(path)["model"])
    opt2 = SGD(net2.parameters(), lr=0.05, momentum=0.9)
    opt2.load_state_dict(mt.load(path)["optimizer"])
    for p, q in zip(net.parameters(), net2.parameters()):
        assert np.array_equal(g.host(opt.state[p]["momentum_buffer"]), g.host(opt2.state[q]["momentum_buffer"]))
