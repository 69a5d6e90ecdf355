"""Two NCCL ranks on two GPUs: the gradient all-reduce that starts bucket by bucket on a side
stream during backward gives bit-identical parameters to the single all-reduce after backward,
eagerly and when the whole step is replayed from a CUDA graph.  Skipped with fewer than 2 GPUs."""
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


@pytest.mark.gpu
def test_bucketed_allreduce_overlap_is_bit_identical(tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    init = f"file://{tmp_path}/rdzv"
    procs = []
    for r in range(2):
        env = dict(os.environ, REPO=ROOT, RANK=str(r), INIT=init, NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=240)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0])
    for p, o in zip(procs, outs):
        assert p.returncode == 0 and "ok" in o, o[-3000:]
