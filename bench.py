"""Benchmark: ResNet-18 (CIFAR variant) training step, global batch 512, fp32 storage with TF32
tensor-core convolutions, SGD lr 0.1 momentum 0.9, data-parallel over N GPUs (one process each).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Under torchrun (N > 1) every rank runs this file; rank 0 prints ONE JSON line.  Synthetic
3x32x32 images ~ N(0,1) and uniform labels stand in for CIFAR-10 (no dataset is read).

`value`  : images/s with the batch already resident in device memory (whole job, all ranks).
`e2e`    : the same step fed from pinned host memory each iteration (H2D of images + labels,
           D2H of the loss) through the package's public API.
`roofline`: the dominant kernel timed alone with CUDA events on its launch stream.
`cpu_baseline` / `--impl reference`: the same ResNet-18 step at batch 64 on the host cores, run by
the reference's own CPU backend when a checkout of the reference is present on the machine
(`baseline/_ref` or `$MYTORCH_REFERENCE`), otherwise by the NumPy restatement of that backend.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GLOBAL_BATCH = 512
SEED = 1003
WORKLOAD = "configs[3]: ResNet-18 CIFAR variant, full training step (fwd+bwd+SGD momentum), global batch 512, 3x32x32"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, f"/tmp/mtb_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [s.strip() for s in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def conv_flops_resnet18(batch):
    """Algorithmic FLOPs (2*M*N*K per GEMM) of every conv and the fc layer, forward only."""
    total, hw, cin = 0, 32, 3
    total += 2 * batch * hw * hw * 64 * cin * 9
    cin = 64
    for si, wd in enumerate((64, 128, 256, 512)):
        for bi in range(2):
            stride = 2 if (si > 0 and bi == 0) else 1
            hw_out = hw // stride
            total += 2 * batch * hw_out * hw_out * wd * cin * 9
            total += 2 * batch * hw_out * hw_out * wd * wd * 9
            if stride != 1 or cin != wd:
                total += 2 * batch * hw_out * hw_out * wd * cin
            cin, hw = wd, hw_out
    total += 2 * batch * 512 * 10
    return total


# --------------------------------------------------------------------------- reference / CPU arm

def cpu_reference_step(sample_batch, steps, warmup):
    """The NumPy oracle's ResNet-18 step on `sample_batch` images, all host threads."""
    from oracle import models as OM

    rng = np.random.default_rng(SEED)
    x = rng.standard_normal((sample_batch, 3, 32, 32)).astype(np.float32)
    t = rng.integers(0, 10, sample_batch).astype(np.int64)
    net = OM.resnet18_cifar(SEED)
    for _ in range(warmup):
        net.train_step(x, t, 0.1, 0.9)
    t0 = time.perf_counter()
    for _ in range(steps):
        net.train_step(x, t, 0.1, 0.9)
    dt = (time.perf_counter() - t0) / steps
    return sample_batch / dt, dt


def blas_threads():
    try:
        from threadpoolctl import threadpool_info

        return max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        return os.cpu_count() or 1


def find_reference():
    """A checkout of the reference (a directory holding its ``mytorch`` package), if one is present:
    ``baseline/_ref`` beside this file, else ``$MYTORCH_REFERENCE``."""
    for cand in (os.path.join(ROOT, "baseline", "_ref"), os.environ.get("MYTORCH_REFERENCE", "")):
        if cand and os.path.isdir(os.path.join(cand, "mytorch")):
            return cand
    return None


def reference_cpu_step(ref_root, sample_batch, steps, warmup):
    """The reference's own CPU backend driven through its public API (nn / autograd / optim) on the
    same ResNet-18 step.  Its package is called ``mytorch``; nothing of this repository is on that path."""
    sys.path.insert(0, ref_root)
    import mytorch.nn as rnn
    import mytorch.nn.functional as RF
    from mytorch.optim import SGD as RSGD
    from mytorch.rand_generator import manual_seed as rseed
    from mytorch.tensor import Tensor as RT

    class Block(rnn.Module):
        def __init__(self, cin, cout, stride):
            super().__init__()
            self.conv1, self.bn1 = rnn.Conv2d(cin, cout, 3, stride, 1, bias=False), rnn.BatchNorm2d(cout)
            self.conv2, self.bn2 = rnn.Conv2d(cout, cout, 3, 1, 1, bias=False), rnn.BatchNorm2d(cout)
            self.downsample = None
            if stride != 1 or cin != cout:
                self.downsample = rnn.Sequential(rnn.Conv2d(cin, cout, 1, stride, 0, bias=False), rnn.BatchNorm2d(cout))
            self.relu = rnn.ReLU()

        def forward(self, x):
            y = self.bn2(self.conv2(self.relu(self.bn1(self.conv1(x)))))
            return self.relu(y + (x if self.downsample is None else self.downsample(x)))

    class Net(rnn.Module):
        def __init__(self):
            super().__init__()
            self.conv1, self.bn1, self.relu = rnn.Conv2d(3, 64, 3, 1, 1, bias=False), rnn.BatchNorm2d(64), rnn.ReLU()
            cin = 64
            for si, wd in enumerate((64, 128, 256, 512)):
                setattr(self, f"layer{si + 1}", rnn.Sequential(Block(cin, wd, 2 if si else 1), Block(wd, wd, 1)))
                cin = wd
            self.fc = rnn.Linear(512, 10)

        def forward(self, x):
            x = self.relu(self.bn1(self.conv1(x)))
            x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
            return self.fc(x.mean(dim=(2, 3)))

    rng = np.random.default_rng(SEED)
    x = rng.standard_normal((sample_batch, 3, 32, 32)).astype(np.float32)
    t = rng.integers(0, 10, sample_batch).astype(np.int64)
    rseed(SEED)
    net = Net()
    opt = RSGD(net.parameters(), lr=0.1, momentum=0.9)

    def step():
        loss = RF.cross_entropy(net(RT(cpu_array=x)), RT(cpu_array=t))
        opt.zero_grad()
        loss.backward()
        opt.step()

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return sample_batch / dt, dt


CPU_SAMPLE_BATCH = 64


def cpu_arm(steps, warmup):
    """(images/s, seconds per step, cpu_baseline dict): the reference itself when a checkout is
    present on this machine, otherwise the NumPy restatement of its CPU backend."""
    ref = find_reference()
    if ref is not None:
        ips, dt = reference_cpu_step(ref, CPU_SAMPLE_BATCH, steps, warmup)
        kind, what = "reference", f"the reference's own CPU backend (checkout at {os.path.relpath(ref, ROOT)})"
    else:
        ips, dt = cpu_reference_step(CPU_SAMPLE_BATCH, steps, warmup)
        kind, what = "port", ("the NumPy restatement of the reference CPU backend (no checkout of the reference on this machine: "
                              "looked in baseline/_ref and $MYTORCH_REFERENCE)")
    return ips, dt, {"value": ips, "unit": "images/s", "cores": blas_threads(), "kind": kind,
                     "sample": f"{steps} full ResNet-18 training step(s) (forward, backward, SGD momentum) at batch {CPU_SAMPLE_BATCH} "
                               f"of the global batch of {GLOBAL_BATCH}, after {warmup} warm-up step(s), with {what}"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 2)), max(0, min(args.warmup, 1))
    ips, dt, cpu = cpu_arm(steps, warmup)
    line = {
        "impl": "reference", "metric": "train_images_per_sec", "value": ips, "unit": "images/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64/f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "parallelism": "cpu", "sample_batch": CPU_SAMPLE_BATCH},
        "cpu_baseline": cpu,
        "e2e": {"value": ips, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- GPU arm

def reference_first_loss(world):
    """First-step loss of this very configuration (seed, batch, initial weights) computed by the
    reference's CPU backend with the batch split into `world` shards (BatchNorm statistics per
    shard, mean of the shard losses); recorded in a fixture because the reference cannot run here."""
    path = os.path.join(ROOT, "tests", "golden", "data_parallel.npz")
    if GLOBAL_BATCH != 512 or not os.path.exists(path):
        return None
    with np.load(path) as gd:
        key = f"c3_b512/w{world}/loss"
        return float(gd[key]) if key in gd else None


def kernel_legs(env, peaks):
    """Time the dominant kernels alone (CUDA events on the launch stream, buffers rotated so that
    every launch reads data that is not in L2).  Returns (roofline dict, per-kernel dict)."""
    import mytorch_b200 as mt
    from mytorch_b200.backends.backend_dispatcher import BackendDispatcher

    op = lambda name: BackendDispatcher.instance().dispatch("cuda", name)
    rng = np.random.default_rng(1)
    from mytorch_b200.backends.cuda.env import Event

    def timed(fn, reps=10, warm=3):
        """seconds per call: CUDA events on the compute stream the kernels are launched on"""
        for i in range(warm):
            fn(i)
        env.synchronize()
        e0, e1 = Event(timing=True), Event(timing=True)
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        env.synchronize()
        return e0.elapsed_ms(e1) / reps * 1e-3

    out = {}
    # dominant conv layer of the step: 64->64 3x3 on 32x32 at the full batch (4 of the 20 convs, 27% of the FLOPs)
    n = GLOBAL_BATCH
    sets = []
    for _ in range(3):  # 3 x (134 MB in + 134 MB out) > 126 MB L2
        x = mt.tensor(rng.standard_normal((n, 64, 32, 32)).astype(np.float32), device="cuda", requires_grad=True)
        dy = mt.tensor(rng.standard_normal((n, 64, 32, 32)).astype(np.float32), device="cuda")
        sets.append((x, dy))
    w = mt.tensor((rng.standard_normal((64, 64, 3, 3)) / 24).astype(np.float32), device="cuda", requires_grad=True)
    flops = 2.0 * n * 32 * 32 * 64 * 64 * 9
    t_f = timed(lambda i: op("conv2d")(sets[i % 3][0], w, None, (1, 1), (1, 1)))
    w.requires_grad = False
    t_d = timed(lambda i: op("conv2d_backward")(sets[i % 3][1], sets[i % 3][0], w, None, (1, 1), (1, 1)))
    w.requires_grad = True
    for x, _ in sets:
        x.requires_grad = False
    t_w = timed(lambda i: op("conv2d_backward")(sets[i % 3][1], sets[i % 3][0], w, None, (1, 1), (1, 1)))
    tf32_peak = peaks["bf16_tflops"] / 2
    out["conv3x3_64_fwd_tflops"] = flops / t_f / 1e12
    out["conv3x3_64_dgrad_tflops"] = flops / t_d / 1e12
    out["conv3x3_64_wgrad_tflops"] = flops / t_w / 1e12
    # BatchNorm forward (3S) / backward (5S) and ReLU on the same activation shape
    x, dy = sets[0]
    S = 4.0 * n * 64 * 32 * 32
    gamma = mt.tensor(np.ones(64, np.float32), device="cuda", requires_grad=True)
    beta = mt.tensor(np.zeros(64, np.float32), device="cuda", requires_grad=True)
    rm, rv = mt.tensor(np.zeros(64, np.float32), device="cuda"), mt.tensor(np.ones(64, np.float32), device="cuda")
    res = {}

    def bn_f(i):
        res["y"], res["m"], res["v"] = op("batch_norm2d")(sets[i % 3][0], gamma, beta, 1e-5, True, 0.1, rm, rv)

    t = timed(bn_f)
    out["bn_fwd_gbs"] = 3 * S / t / 1e9
    t = timed(lambda i: op("batch_norm2d_backward")(sets[i % 3][1], res["m"], res["v"], sets[i % 3][0], gamma, beta, 1e-5))
    out["bn_bwd_gbs"] = 5 * S / t / 1e9
    t = timed(lambda i: op("relu")(sets[i % 3][0]))
    out["relu_fwd_gbs"] = 2 * S / t / 1e9
    del sets, x, dy, res
    # configs[1]: conv 64->64 3x3 on 128x56x56, forward + dgrad + wgrad (103 MB in, 103 MB out per pass)
    n1 = 128
    big = rng.standard_normal((n1, 64, 56, 56)).astype(np.float32)
    c1 = [(mt.tensor(big, device="cuda", requires_grad=True), mt.tensor(big[::-1].copy(), device="cuda")) for _ in range(2)]
    flops1 = 2.0 * n1 * 56 * 56 * 64 * 64 * 9
    bias = mt.tensor(np.zeros(64, np.float32), device="cuda")
    t_f = timed(lambda i: op("conv2d")(c1[i % 2][0], w, bias, (1, 1), (1, 1)))
    w.requires_grad = False
    t_d = timed(lambda i: op("conv2d_backward")(c1[i % 2][1], c1[i % 2][0], w, None, (1, 1), (1, 1)))
    w.requires_grad = True
    for xx, _ in c1:
        xx.requires_grad = False
    t_w = timed(lambda i: op("conv2d_backward")(c1[i % 2][1], c1[i % 2][0], w, None, (1, 1), (1, 1)))
    out["config1_conv56_fwd_tflops"] = flops1 / t_f / 1e12
    out["config1_conv56_dgrad_tflops"] = flops1 / t_d / 1e12
    out["config1_conv56_wgrad_tflops"] = flops1 / t_w / 1e12
    del c1
    # a late layer: 256->256 3x3 on 8x8 at the full batch (im2col-mode kernels; 33.5 MB per tensor, five sets rotate past L2)
    late = []
    for _ in range(5):
        late.append((mt.tensor(rng.standard_normal((n, 256, 8, 8)).astype(np.float32), device="cuda", requires_grad=True),
                     mt.tensor(rng.standard_normal((n, 256, 8, 8)).astype(np.float32), device="cuda")))
    w256 = mt.tensor((rng.standard_normal((256, 256, 3, 3)) / 48).astype(np.float32), device="cuda", requires_grad=True)
    flops256 = 2.0 * n * 8 * 8 * 256 * 256 * 9
    t_f = timed(lambda i: op("conv2d")(late[i % 5][0], w256, None, (1, 1), (1, 1)))
    w256.requires_grad = False
    t_d = timed(lambda i: op("conv2d_backward")(late[i % 5][1], late[i % 5][0], w256, None, (1, 1), (1, 1)))
    w256.requires_grad = True
    for xx, _ in late:
        xx.requires_grad = False
    t_w = timed(lambda i: op("conv2d_backward")(late[i % 5][1], late[i % 5][0], w256, None, (1, 1), (1, 1)))
    out["conv3x3_256_8x8_fwd_tflops"] = flops256 / t_f / 1e12
    out["conv3x3_256_8x8_dgrad_tflops"] = flops256 / t_d / 1e12
    out["conv3x3_256_8x8_wgrad_tflops"] = flops256 / t_w / 1e12
    del late, w256
    # configs[2]: BatchNorm2d(128) -> ReLU -> MaxPool2d(2,2) on 256x128x56x56 (S = 411 MB >> L2), forward and backward
    big2 = (0.5 + 2.0 * rng.standard_normal((64, 128, 56, 56))).astype(np.float32)
    x2 = mt.tensor(np.concatenate([big2] * 4, axis=0), device="cuda", requires_grad=True)
    S2 = 4.0 * 256 * 128 * 56 * 56
    g2 = mt.tensor(np.ones(128, np.float32), device="cuda", requires_grad=True)
    b2 = mt.tensor(np.zeros(128, np.float32), device="cuda", requires_grad=True)
    rm2, rv2 = mt.tensor(np.zeros(128, np.float32), device="cuda"), mt.tensor(np.ones(128, np.float32), device="cuda")
    r2 = {}

    def bn2_f(i):
        r2["y"], r2["m"], r2["v"] = op("batch_norm2d")(x2, g2, b2, 1e-5, True, 0.1, rm2, rv2)

    out["config2_bn_fwd_gbs"] = 3 * S2 / timed(bn2_f, reps=5) / 1e9
    out["config2_bn_bwd_gbs"] = 5 * S2 / timed(lambda i: op("batch_norm2d_backward")(r2["y"], r2["m"], r2["v"], x2, g2, b2, 1e-5), reps=5) / 1e9
    out["config2_relu_fwd_gbs"] = 2 * S2 / timed(lambda i: r2.__setitem__("r", op("relu")(r2["y"])), reps=5) / 1e9
    out["config2_relu_bwd_gbs"] = 3 * S2 / timed(lambda i: op("relu_backward")(x2, r2["y"]), reps=5) / 1e9

    def pool_f(i):
        r2["p"] = op("max_pool2d")(r2["r"], (2, 2), (2, 2), (0, 0))

    # forward: read S, write S/4 values + S/8 tie mask (uint16 per output); backward: read S/4 + S/8, write S
    out["config2_maxpool_fwd_gbs"] = 1.375 * S2 / timed(pool_f, reps=5) / 1e9
    dyp = mt.tensor(big2[:, :, ::2, ::2].repeat(4, axis=0).copy(), device="cuda")
    out["config2_maxpool_bwd_gbs"] = 1.375 * S2 / timed(lambda i: op("max_pool2d_backward")(dyp, r2["p"], r2["r"], (2, 2), (2, 2), (0, 0)), reps=5) / 1e9
    del r2, x2, dyp
    roof = {"bound": "tensor", "kernel": "conv2d forward 64->64 3x3 s1 p1 on 512x32x32 (dominant layer shape of the step)",
            "achieved": out["conv3x3_64_fwd_tflops"], "peak": tf32_peak, "unit": "TFLOP/s", "frac": out["conv3x3_64_fwd_tflops"] / tf32_peak,
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel and shape, from the ncu
            # capture summarised in profiles/ (134.5 MB read + 83.9 MB written; algorithmic: 134 + 134 MB,
            # part of the output is still in L2 when the kernel ends)
            "traffic": 218.4e6, "algorithmic_flops_per_launch": flops,
            "peak_note": f"TF32 dense = half of the {peaks['source']} bf16 burst figure ({peaks['bf16_tflops']} TFLOP/s); "
                         f"HBM figures in `kernels` are against {peaks['hbm_gbs']} GB/s ({peaks['source']})"}
    out["hbm_frac"] = {k: out[k] / peaks["hbm_gbs"] for k in out if k.endswith("_gbs")}
    out["tf32_frac"] = {k: out[k] / tf32_peak for k in out if k.endswith("_tflops")}
    return roof, out


def profile_leg(env, name, iters=3):
    """One operator at a benchmark shape, a few launches, nothing else on the device: the command
    profiled with ncu for the summaries under profiles/ (kept small so that a full-counter capture ends
    by itself).  conv64: 64->64 3x3 on 512x32x32 forward, forward with BatchNorm statistics, dgrad,
    wgrad; wgrad256: weight gradient of 256->256 3x3 on 512x8x8 (im2col kernel); pool: 2x2/2 max-pool
    forward and backward on 256x128x56x56; bn64: BatchNorm forward / backward on 512x64x32x32; bn64add: the
    same shape through the BatchNorm + shortcut add + ReLU operator of a residual block's tail."""
    import mytorch_b200 as mt
    from mytorch_b200.backends.backend_dispatcher import BackendDispatcher

    op = lambda n: BackendDispatcher.instance().dispatch("cuda", n)
    rng = np.random.default_rng(2)
    dev = lambda a, grad=False: mt.tensor(a.astype(np.float32), device="cuda", requires_grad=grad)
    if name in ("conv64", "bn64", "bn64add"):
        x, dy = dev(rng.standard_normal((512, 64, 32, 32)), True), dev(rng.standard_normal((512, 64, 32, 32)))
        if name == "conv64":
            w = dev(rng.standard_normal((64, 64, 3, 3)) / 24, True)
            for _ in range(iters):
                op("conv2d")(x, w, None, (1, 1), (1, 1))
                op("conv2d")(x, w, None, (1, 1), (1, 1), bn_stats=True)
                op("conv2d_backward")(dy, x, w, None, (1, 1), (1, 1))
        elif name == "bn64":
            g, b = dev(np.ones(64), True), dev(np.zeros(64), True)
            for _ in range(iters):
                y, m, v = op("batch_norm2d")(x, g, b, 1e-5, True, 0.1, None, None)
                op("batch_norm2d_backward")(dy, m, v, x, g, b, 1e-5)
        else:
            g, b = dev(np.ones(64), True), dev(np.zeros(64), True)
            res = dev(rng.standard_normal((512, 64, 32, 32)), True)
            for _ in range(iters):
                y, m, v = op("batch_norm2d_add_relu")(x, res, g, b, 1e-5, True, 0.1, None, None)
                op("batch_norm2d_add_relu_backward")(dy, m, v, x, res, g, b, 1e-5)
    elif name == "wgrad256":
        x, dy = dev(rng.standard_normal((512, 256, 8, 8))), dev(rng.standard_normal((512, 256, 8, 8)))
        w = dev(rng.standard_normal((256, 256, 3, 3)) / 48, True)
        for _ in range(iters):
            op("conv2d_backward")(dy, x, w, None, (1, 1), (1, 1))
    elif name == "pool":
        x = dev(np.concatenate([rng.standard_normal((64, 128, 56, 56)).astype(np.float32)] * 4, axis=0))
        dy = dev(rng.standard_normal((256, 128, 28, 28)))
        for _ in range(iters):
            y = op("max_pool2d")(x, (2, 2), (2, 2), (0, 0))
            op("max_pool2d_backward")(dy, y, x, (2, 2), (2, 2), (0, 0))
    else:
        sys.exit(f"unknown leg {name}")
    env.synchronize()
    status = env.tensor_core_status()
    print(json.dumps({"leg": name, "iterations": iters, "tensor_core_status": status}))


def run_gpu_arm(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch = dist = None
    if world > 1:  # PyTorch only carries the NCCL process group; one GPU runs without it
        import torch
        import torch.distributed as dist
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            sys.exit(f"--gpus {args.gpus} needs torchrun: python -m torch.distributed.run --nproc-per-node {args.gpus} bench.py ...")
    if world > 1:
        torch.cuda.set_device(local)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))

    import mytorch_b200 as mt
    import mytorch_b200.nn.functional as F
    from mytorch_b200.backends.cuda.env import CudaEnv, Event, PinnedBuffer
    from mytorch_b200.cuda_graph import StepGraph
    from mytorch_b200.examples.models import ResNet18Cifar
    from mytorch_b200.optim import SGD
    from mytorch_b200.parallel import DataParallel, shard_bounds

    env = CudaEnv.instance()
    env.set_device(local)
    dev = f"cuda:{local}"
    peaks = measured_peaks()

    rng = np.random.default_rng(SEED)
    x_all = rng.standard_normal((GLOBAL_BATCH, 3, 32, 32)).astype(np.float32)
    t_all = rng.integers(0, 10, GLOBAL_BATCH).astype(np.int64)
    lo, hi = shard_bounds(GLOBAL_BATCH, rank, world)
    local_batch = hi - lo
    # a few distinct host batches in pinned memory for the end-to-end leg
    pinned = []
    for s in range(4):
        px, pt = PinnedBuffer((local_batch, 3, 32, 32), np.float32), PinnedBuffer((local_batch,), np.int64)
        px.array[...] = np.roll(x_all, s, axis=0)[lo:hi]
        pt.array[...] = np.roll(t_all, s, axis=0)[lo:hi]
        pinned.append((px, pt))
    host_x, host_t = [p[0].array for p in pinned], [p[1].array for p in pinned]

    mt.manual_seed(SEED)
    net = ResNet18Cifar()
    net.to(dev)
    dp = DataParallel(net, buckets=args.grad_buckets)
    opt = SGD(net.parameters(), lr=0.1, momentum=0.9)
    xs = mt.tensor(x_all[lo:hi], device=dev)
    ts = mt.tensor(t_all[lo:hi], device=dev)

    def step():
        loss = F.cross_entropy(dp(xs), ts)
        opt.zero_grad()
        loss.backward()
        dp.reduce_gradients()
        opt.step()
        return loss

    def barrier():
        env.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
    first_loss = step().item()
    if world > 1:  # the job's loss is the mean of the shard losses
        fl = torch.tensor([first_loss], device=dev)
        dist.all_reduce(fl)
        first_loss = float(fl.item()) / world
    loss_ref = reference_first_loss(world)
    step()
    env.synchronize()
    runner = None
    if not args.no_graph:
        before = env.lib.launches
        sg = StepGraph(step, [xs, ts])
        sg.capture()
        calls_per_step = env.lib.launches - before
        runner = sg
    else:
        before = env.lib.launches
        step()
        calls_per_step = env.lib.launches - before

    def run_resident():
        if runner is not None:
            runner.replay()
        else:
            step()

    def run_e2e(i):
        if runner is not None:
            # batch i was staged during step i-1; stage batch i+1 now so that its copy overlaps this step
            runner.replay(prefetched=True)
            runner.prefetch([host_x[(i + 1) % 4], host_t[(i + 1) % 4]])
            return runner.result.item()
        from mytorch_b200.backends.cuda.ops import upload_into

        upload_into(xs, host_x[i % 4])
        upload_into(ts, host_t[i % 4])
        return step().item()

    def timed_region(body, steps):
        """milliseconds for `steps` steps: CUDA events on the compute stream, barrier + synchronise on both
        sides, the maximum over ranks"""
        barrier()
        e0, e1 = Event(timing=True), Event(timing=True)
        e0.record()
        for i in range(steps):
            body(i)
        e1.record()
        barrier()
        elapsed = e0.elapsed_ms(e1)
        if world > 1:
            ms = torch.tensor([elapsed], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            elapsed = float(ms.item())
        return elapsed

    for _ in range(max(args.warmup, 3)):
        run_resident()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # the timed region of K steps is short (tens of milliseconds), so it is repeated and the median
    # region is reported, with the spread beside it; the clock sampler runs across all repeats
    resident_ms = [timed_region(lambda i: run_resident(), args.steps) for _ in range(args.repeats)]
    if runner is not None:
        runner.prefetch([host_x[0], host_t[0]])
    for i in range(2):
        run_e2e(i)
    e2e_all = [timed_region(lambda i: run_e2e(i + 2), args.steps) for _ in range(args.repeats)]
    clocks = sampler.stop() if rank == 0 else None
    last_loss = run_e2e(args.steps + 2)

    total_ms, e2e_ms = statistics.median(resident_ms), statistics.median(e2e_all)
    ms_per_step = total_ms / args.steps
    value = GLOBAL_BATCH / (ms_per_step * 1e-3)
    e2e_value = GLOBAL_BATCH / (e2e_ms / args.steps * 1e-3)
    tc_status = env.tensor_core_status()
    if tc_status != 0:
        sys.exit(f"a bounded wait inside a tensor-core kernel ran out (status {tc_status}): results are not valid")
    step_flops = 3 * conv_flops_resnet18(GLOBAL_BATCH) - 2 * GLOBAL_BATCH * 32 * 32 * 64 * 27  # stem dgrad is not executed

    roof, kernels, cpu = None, None, None
    if rank == 0 and world == 1 and not args.skip_legs:
        roof, kernels = kernel_legs(env, peaks)
        try:
            import torch

            a = torch.randn(8192, 8192, device=dev)
            b = torch.randn(8192, 8192, device=dev)
            torch.backends.cuda.matmul.allow_tf32 = True
            best = 1e9
            for _ in range(6):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                torch.matmul(a, b)
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1))
            kernels["cublas_tf32_8192_tflops"] = 2 * 8192 ** 3 / (best * 1e-3) / 1e12
        except Exception as e:  # measurement aid only
            kernels["cublas_tf32_8192_tflops"] = f"unavailable: {e}"
        _, _, cpu = cpu_arm(1, 0)
        tc_status = env.tensor_core_status()
        if tc_status != 0:
            sys.exit(f"a bounded wait inside a tensor-core kernel ran out in the single-kernel legs (status {tc_status})")

    if rank == 0:
        line = {
            "metric": "train_images_per_sec", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "tf32 (fp32 storage, fp32 accumulate)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "per_gpu_batch": local_batch, "parallelism": f"dp{world}", "grad_buckets": args.grad_buckets if world > 1 else None,
                       "cuda_graph": not args.no_graph,
                       "l2": "no flush: one step streams ~1.3 GB of activations per pass, 10x the 126 MB L2"},
            "step_tflops": step_flops / (ms_per_step * 1e-3) / 1e12,
            "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": int(host_x[0].nbytes + host_t[0].nbytes) * world,
                    "d2h_bytes_per_step": 4 * world},
            "gpu_launches": calls_per_step * args.steps,
            "gpu_launches_note": "C-ABI calls per step x steps; each call enqueues 1-3 kernels of libmytorch_b200.so",
            "loss_first": first_loss, "loss_first_ref": loss_ref, "loss_first_rel_err": None if loss_ref is None else abs(first_loss - loss_ref) / abs(loss_ref),
            "loss_last": last_loss, "tensor_core_status": tc_status,
            "repeats": {"n": args.repeats, "ms_per_step_min": min(resident_ms) / args.steps, "ms_per_step_max": max(resident_ms) / args.steps,
                        "e2e_ms_per_step_min": min(e2e_all) / args.steps, "e2e_ms_per_step_max": max(e2e_all) / args.steps,
                        "reported": "median of the repeated K-step regions"},
            "clocks": clocks, "roofline": roof, "kernels": kernels, "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    if world > 1:
        # Tearing down a NCCL process group whose collectives were captured in a CUDA graph that is
        # still alive blocks in this PyTorch/NCCL combination; finish with a barrier and leave the
        # process without running the communicator's destructor.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    global GLOBAL_BATCH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--repeats", type=int, default=5, help="how many times the timed region of K steps is repeated (the median is reported)")
    ap.add_argument("--no-graph", action="store_true", help="launch every operator eagerly instead of replaying a CUDA graph")
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH,
                    help="profiling aid: run the step at another global batch (the benchmark configuration is 512)")
    ap.add_argument("--grad-buckets", type=int, default=1,
                    help="gradient all-reduce buckets (N>1): 1 = one all-reduce after backward, more = start each "
                         "bucket on a side stream as soon as backward has finished its gradients")
    ap.add_argument("--skip-legs", action="store_true", help="skip the single-kernel roofline and CPU-baseline legs")
    ap.add_argument("--leg", default=None, choices=["conv64", "wgrad256", "pool", "bn64", "bn64add"],
                    help="run one operator at a benchmark shape for a few launches and exit (the small command profiled with ncu)")
    ap.add_argument("--only-legs", action="store_true",
                    help="run only the single-kernel legs (conv fwd/dgrad/wgrad, BatchNorm, ReLU) and print their JSON; "
                         "this is the command profiled with ncu for the summaries under profiles/")
    args = ap.parse_args()
    GLOBAL_BATCH = args.global_batch
    if args.leg:
        from mytorch_b200.backends.cuda.env import CudaEnv

        profile_leg(CudaEnv.instance(), args.leg)
    elif args.only_legs:
        from mytorch_b200.backends.cuda.env import CudaEnv

        roof, kernels = kernel_legs(CudaEnv.instance(), measured_peaks())
        print(json.dumps({"roofline": roof, "kernels": kernels}))
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
