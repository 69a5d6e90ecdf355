"""Data-parallel host logic on CPU: two gloo ranks average their gradients through the flat
bucket, and a rank that never joins is reported by a timeout instead of a hang."""
import os
import subprocess
import sys
import textwrap

from conftest import ROOT

WORKER = textwrap.dedent("""
    import os, sys, datetime
    import numpy as np
    import torch.distributed as dist
    sys.path.insert(0, os.environ["REPO"])
    import mytorch_b200 as mt, mytorch_b200.nn as nn
    from mytorch_b200.parallel import DataParallel, shard_batch
    dist.init_process_group("gloo", init_method=os.environ["INIT"], rank=int(os.environ["RANK"]), world_size=2,
                            timeout=datetime.timedelta(seconds=60))
    rank = dist.get_rank()
    mt.manual_seed(3 + rank)            # different init per rank on purpose
    net = nn.Sequential(nn.Linear(5, 4), nn.Linear(4, 3))
    dp = DataParallel(net)
    dp.broadcast_parameters(0)
    mt.manual_seed(3)
    ref = nn.Sequential(nn.Linear(5, 4), nn.Linear(4, 3))
    for a, b in zip(net.parameters(), ref.parameters()):
        assert np.array_equal(a._numpy(), b._numpy())
    full = np.arange(12 * 2, dtype=np.float32).reshape(12, 2)
    mine = shard_batch(full, rank, 2)
    assert mine.shape == (6, 2) and mine[0, 0] == rank * 12
    for i, p in enumerate(net.parameters()):
        p.grad = mt.tensor(np.full(p.shape, float((rank + 1) * (i + 1)), np.float32))
    dp.reduce_gradients()
    for i, p in enumerate(net.parameters()):
        assert p.grad.shape == p.shape and np.allclose(p.grad._numpy(), 1.5 * (i + 1)), (i, p.grad._numpy())
    dist.destroy_process_group()
    print("ok", rank)
""")


def _spawn(code, rank, init, extra=None):
    env = dict(os.environ, REPO=ROOT, RANK=str(rank), INIT=init, **(extra or {}))
    return subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)


def test_two_rank_gradient_average(tmp_path):
    init = f"file://{tmp_path}/rdzv"
    procs = [_spawn(WORKER, r, init) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        assert "ok" in o


BUCKETED = textwrap.dedent("""
    import os, sys, datetime
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, os.environ["REPO"])
    import mytorch_b200 as mt, mytorch_b200.nn as nn, mytorch_b200.nn.functional as F
    from mytorch_b200.parallel import DataParallel, split_into_buckets
    dist.init_process_group("gloo", init_method=os.environ["INIT"], rank=int(os.environ["RANK"]), world_size=2,
                            timeout=datetime.timedelta(seconds=60))
    rank = dist.get_rank()

    # the CPU backend has storage operators only; the host logic under test needs a differentiable
    # graph, so NumPy stand-ins from the oracle are registered for the three operators it uses
    from mytorch_b200.backends.backend_dispatcher import BackendDispatcher
    from oracle import ops as O
    reg = BackendDispatcher.instance().register_backend_function
    T = lambda a: mt.tensor(np.asarray(a, np.float32))
    N = lambda t: t._numpy()
    reg("cpu", "linear")(lambda x, w, b: T(O.linear_forward(N(x), N(w), N(b))))
    reg("cpu", "linear_backward")(lambda dy, x, w, b: [T(g) for g in O.linear_backward(N(dy), N(x), N(w), True)])
    reg("cpu", "relu")(lambda x: T(O.relu_forward(N(x))))
    reg("cpu", "relu_backward")(lambda dy, x: [T(O.relu_backward(N(dy), N(x)))])
    reg("cpu", "cross_entropy")(lambda z, t: T(O.cross_entropy_forward(N(z), N(t))).reshape((1,)))
    reg("cpu", "cross_entropy_backward")(lambda dy, z, t: [T(O.cross_entropy_backward(N(dy).reshape(()), N(z), N(t)))])

    def build():
        mt.manual_seed(11)
        return nn.Sequential(nn.Linear(6, 8), nn.ReLU(), nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 4))

    rng = np.random.default_rng(100 + rank)
    x = mt.tensor(rng.standard_normal((5, 6)).astype(np.float32))
    t = mt.tensor(rng.integers(0, 4, 5).astype(np.int64))

    plain = build()                      # local gradients, averaged by hand below
    F.cross_entropy(plain(x), t).backward()
    want = []
    for p in plain.parameters():
        g = torch.from_numpy(p.grad._numpy().copy())
        dist.all_reduce(g)
        want.append(g.numpy() / 2)

    net = build()
    dp = DataParallel(net, buckets=3)
    assert len(dp.buckets) == 3
    started = []
    launch = dp._launch_bucket
    dp._launch_bucket = lambda b, stream=None: (started.append(b), launch(b, stream))[1]
    for step in range(2):                # the second pass checks that the counters were re-armed
        for p in net.parameters():
            p.grad = None
        del started[:]
        loss = F.cross_entropy(dp(x), t)
        loss.backward()
        # every bucket left during backward, the deepest layers' first
        assert started[0] == 0 and sorted(started) == [0, 1, 2], started
        dp.reduce_gradients()
        assert len(started) == 3, started
        for p, w in zip(net.parameters(), want):
            assert p.grad.shape == p.shape and np.allclose(p.grad._numpy(), w, rtol=1e-6, atol=1e-7)
    groups = split_into_buckets(list(net.parameters()), 3)
    assert [id(p) for g in groups for p in g] == [id(p) for p in list(net.parameters())[::-1]]
    dist.destroy_process_group()
    print("ok", rank)
""")


def test_bucketed_reduce_starts_during_backward(tmp_path):
    init = f"file://{tmp_path}/rdzv3"
    procs = [_spawn(BUCKETED, r, init) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        assert "ok" in o


LONELY = textwrap.dedent("""
    import os, sys, datetime
    import torch.distributed as dist
    try:
        dist.init_process_group("gloo", init_method=os.environ["INIT"], rank=0, world_size=2,
                                timeout=datetime.timedelta(seconds=3))
    except Exception as e:
        print("rendezvous failed:", type(e).__name__)
        sys.exit(7)
""")


def test_missing_rank_is_a_timeout_not_a_hang(tmp_path):
    p = _spawn(LONELY, 0, f"file://{tmp_path}/rdzv2")
    out = p.communicate(timeout=120)[0]
    assert p.returncode == 7 and "rendezvous failed" in out, out
