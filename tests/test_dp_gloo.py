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
