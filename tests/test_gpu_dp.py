"""Data parallelism against the reference.

The reference has no distributed code, so the multi-GPU oracle is the reference's CPU backend
emulating sharded data parallelism (tests/golden/make_golden.py, ``sharded_step``): every shard of
the batch runs through the same initial weights with BatchNorm statistics of its own shard, the
shard gradients are averaged and one SGD step is taken.  Two checks against those fixtures:

* on one GPU, the shards run one after the other and their gradients are averaged on the host
  (same arithmetic as the all-reduce, no NCCL involved);
* on two GPUs, two NCCL ranks run ``DataParallel`` and the averaged gradients and updated
  parameters of both ranks are compared with the fixture (skipped with fewer than 2 GPUs).

A third test checks that the all-reduce started bucket by bucket on a side stream during backward
gives bit-identical parameters to the single all-reduce after backward, eagerly and from a CUDA graph."""
import os
import subprocess
import sys
import textwrap

import pytest

from conftest import ROOT

WORKER = textwrap.dedent("""
    import os, sys, datetime
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, os.environ["REPO"])
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=os.environ["INIT"], rank=rank, world_size=2,
                            timeout=datetime.timedelta(seconds=120), device_id=torch.device(f"cuda:{rank}"))
    import mytorch_b200 as mt, mytorch_b200.nn.functional as F
    from mytorch_b200.cuda_graph import StepGraph
    from mytorch_b200.examples.models import ResNet18Cifar
    from mytorch_b200.optim import SGD
    from mytorch_b200.parallel import DataParallel

    dev = f"cuda:{rank}"
    rng = np.random.default_rng(7 + rank)
    x = mt.tensor(rng.standard_normal((16, 3, 32, 32)).astype(np.float32), device=dev)
    t = mt.tensor(rng.integers(0, 10, 16).astype(np.int64), device=dev)

    def run(buckets, graph):
        mt.manual_seed(5)
        net = ResNet18Cifar(widths=(16, 32, 64, 64))
        net.to(dev)
        dp = DataParallel(net, buckets=buckets)
        assert len(dp.buckets) == buckets
        opt = SGD(net.parameters(), lr=0.05, momentum=0.9)

        def step():
            loss = F.cross_entropy(dp(x), t)
            opt.zero_grad()
            loss.backward()
            dp.reduce_gradients()
            opt.step()
            return loss

        step(); step()
        if graph:
            sg = StepGraph(step, [x, t])
            sg.capture()
            for _ in range(3):
                sg.replay()
        else:
            for _ in range(3):
                step()
        torch.cuda.synchronize()
        return [p.detach().to("cpu")._numpy().copy() for p in net.parameters()]

    base = run(1, False)
    for buckets, graph in ((3, False), (3, True)):
        got = run(buckets, graph)
        for a, b in zip(base, got):
            assert np.array_equal(a, b), (buckets, graph, float(np.abs(a - b).max()))
    # both replicas hold the same parameters after averaged steps
    mine = torch.from_numpy(np.concatenate([a.reshape(-1) for a in base])).cuda()
    other = mine.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(mine, other)
    print("ok", rank, flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)   # a captured graph still holds NCCL work: skip the process-group teardown
""")


def _run_two_ranks(worker, tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    init = f"file://{tmp_path}/rdzv"
    procs = []
    for r in range(2):
        env = dict(os.environ, REPO=ROOT, RANK=str(r), INIT=init, NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, "-c", worker], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=240)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0])
    for p, o in zip(procs, outs):
        assert p.returncode == 0 and "ok" in o, o[-3000:]


@pytest.mark.gpu
def test_bucketed_allreduce_overlap_is_bit_identical(tmp_path):
    _run_two_ranks(WORKER, tmp_path)


# Sharded steps of the reduced-width ResNet: shards of 8 (world 2) or 4 (world 4) images through
# 17 ReLU layers of 16..64 channels.  The loss depends on the forward pass only (5e-3); the averaged
# gradient is compared in relative L2 over the whole vector, like the other small-model fixtures.
DP_LOSS_TOL = 5e-3
DP_GRAD_TOL = 0.15


def _dp_small_inputs():
    import numpy as np

    rng = np.random.default_rng(2002)
    return rng.standard_normal((16, 3, 32, 32)).astype(np.float32), rng.integers(0, 10, 16).astype(np.int64)


def _summary_error(gd, prefix, named):
    import numpy as np

    from conftest import summarize

    num = den = 0.0
    for name, arr in named:
        ref = gd[f"{prefix}/{name}/sample"]
        num += float(np.sum((summarize(arr)[1] - ref) ** 2))
        den += float(np.sum(ref ** 2))
    return (num / max(den, 1e-60)) ** 0.5


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_sharded_step_on_one_gpu_matches_reference_emulation(world):
    import numpy as np

    import gpu_util as g
    import mytorch_b200 as mt
    import mytorch_b200.nn.functional as F
    from conftest import load_golden
    from mytorch_b200.examples.models import ResNet18Cifar
    from mytorch_b200.optim import SGD
    from mytorch_b200.parallel import shard_bounds

    gd = load_golden("data_parallel")
    x, t = _dp_small_inputs()
    losses, sums = [], None
    for r in range(world):
        lo, hi = shard_bounds(16, r, world)
        mt.manual_seed(2002)
        net = ResNet18Cifar((16, 32, 64, 64))
        net.to(g.DEV)
        loss = F.cross_entropy(net(g.dev(x[lo:hi])), g.dev(t[lo:hi]))
        loss.backward()
        losses.append(loss.item())
        grads = [(k, g.host(v.grad).astype(np.float64)) for k, v in net.named_parameters()]
        sums = grads if sums is None else [(k, a + b) for (k, a), (_, b) in zip(sums, grads)]
    tag = f"dp_small/w{world}"
    assert np.allclose(losses, gd[f"{tag}/shard_losses"], rtol=DP_LOSS_TOL, atol=0)
    avg = [(k, (a / world).astype(np.float32)) for k, a in sums]
    assert _summary_error(gd, f"{tag}/grad", avg) < DP_GRAD_TOL
    mt.manual_seed(2002)
    net = ResNet18Cifar((16, 32, 64, 64))
    net.to(g.DEV)
    opt = SGD(net.parameters(), lr=0.1, momentum=0.9)
    for (k, p), (_, a) in zip(net.named_parameters(), avg):
        p.grad = g.dev(a)
    opt.step()
    assert _summary_error(gd, f"{tag}/param", [(k, g.host(v.detach())) for k, v in net.named_parameters()]) < DP_GRAD_TOL


DP_WORKER = textwrap.dedent("""
    import os, sys, datetime
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, os.environ["REPO"]); sys.path.insert(0, os.path.join(os.environ["REPO"], "tests"))
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=os.environ["INIT"], rank=rank, world_size=2,
                            timeout=datetime.timedelta(seconds=120), device_id=torch.device(f"cuda:{rank}"))
    import mytorch_b200 as mt, mytorch_b200.nn.functional as F
    from conftest import load_golden
    from test_gpu_dp import _dp_small_inputs, _summary_error, DP_LOSS_TOL, DP_GRAD_TOL
    from mytorch_b200.examples.models import ResNet18Cifar
    from mytorch_b200.optim import SGD
    from mytorch_b200.parallel import DataParallel
    from mytorch_b200.backends.cuda.env import CudaEnv

    gd = load_golden("data_parallel")
    dev = f"cuda:{rank}"
    x, t = _dp_small_inputs()
    mt.manual_seed(2002)
    net = ResNet18Cifar((16, 32, 64, 64))
    net.to(dev)
    dp = DataParallel(net)
    opt = SGD(net.parameters(), lr=0.1, momentum=0.9)
    loss = F.cross_entropy(dp(mt.tensor(dp.shard(x), device=dev)), mt.tensor(dp.shard(t), device=dev))
    opt.zero_grad()
    loss.backward()
    dp.reduce_gradients()
    mine = loss.item()
    assert abs(mine - gd["dp_small/w2/shard_losses"][rank]) < DP_LOSS_TOL * abs(mine)
    both = torch.tensor([mine], device=dev)
    dist.all_reduce(both)
    assert abs(both.item() / 2 - float(gd["dp_small/w2/loss"])) < DP_LOSS_TOL * float(gd["dp_small/w2/loss"])
    err = _summary_error(gd, "dp_small/w2/grad", [(k, v.grad.to("cpu")._numpy()) for k, v in net.named_parameters()])
    assert err < DP_GRAD_TOL, err
    opt.step()
    err = _summary_error(gd, "dp_small/w2/param", [(k, v.detach().to("cpu")._numpy()) for k, v in net.named_parameters()])
    assert err < DP_GRAD_TOL, err
    assert CudaEnv.instance().tensor_core_status() == 0
    print("ok", rank, flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()
""")


@pytest.mark.gpu
def test_two_nccl_ranks_match_reference_sharded_emulation(tmp_path):
    _run_two_ranks(DP_WORKER, tmp_path)
