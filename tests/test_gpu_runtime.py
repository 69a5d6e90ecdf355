"""The runtime half of the C ABI: memory pool, copies, streams, events, graph capture with pool ownership."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _env():
    from mytorch_b200.backends.cuda.env import CudaEnv

    return CudaEnv.instance()


def test_pool_reuses_addresses_and_counts_bytes():
    env = _env()
    lib = env.lib
    env.synchronize()
    base_use, base_res = lib.pool_in_use_bytes(), lib.pool_reserved_bytes()
    size = 37 << 16                         # a size class (64 KiB granules above 1 MiB) no earlier test left behind
    a = lib.malloc(size)
    b = lib.malloc(size)
    assert a != b and lib.pool_in_use_bytes() == base_use + 2 * size
    lib.free(a)
    c = lib.malloc(size - 4096)            # a slightly smaller request takes the freed block
    assert c == a
    small = lib.malloc(100)
    assert lib.pool_in_use_bytes() == base_use + 2 * size + 512
    for p in (b, c, small):
        lib.free(p)
    assert lib.pool_in_use_bytes() == base_use and lib.pool_reserved_bytes() >= base_res
    from mytorch_b200.backends.cuda.env import NativeError

    with pytest.raises(NativeError, match="not allocated by mtb_malloc"):
        lib.free(12345)


def test_copies_streams_and_events_round_trip():
    from mytorch_b200.backends.cuda.env import Event, PinnedBuffer

    env = _env()
    lib = env.lib
    n = 1 << 20
    src, dst = PinnedBuffer((n,), np.float32), PinnedBuffer((n,), np.float32)
    src.array[...] = np.arange(n, dtype=np.float32)
    dst.array[...] = 0
    d1, d2 = lib.malloc(4 * n), lib.malloc(4 * n)
    side = env.new_stream()
    e0, e1, done = Event(timing=True), Event(timing=True), Event()
    e0.record(side)
    lib.memcpy_h2d_async(d1, src.ptr, 4 * n, side)
    lib.scale_f32(d2, d1, n, 2.0, side)                     # a kernel of the library on the side stream
    e1.record(side)
    done.record(side)
    lib.stream_wait_event(env.stream(), done.handle)       # the compute stream continues after the side stream
    lib.memcpy_d2h_async(dst.ptr, d2, 4 * n, env.stream())
    lib.stream_synchronize(env.stream())
    assert np.array_equal(dst.array, 2 * src.array)
    assert 0 < e0.elapsed_ms(e1) < 1000
    lib.memset_async(d1, 0, 4 * n, env.stream())
    lib.memcpy_d2d_async(d2, d1, 4 * n, env.stream())
    lib.memcpy_d2h_async(dst.ptr, d2, 4 * n, env.stream())
    env.synchronize()
    assert not dst.array.any()
    lib.free(d1)
    lib.free(d2)
    lib.stream_destroy(side)


def test_graph_owns_the_blocks_it_captured():
    """Memory handed out during a capture stays with the graph: after the capture, a block the step
    freed is not given to anybody else, so replays cannot overwrite a live tensor; destroying the
    graph returns it to the pool."""
    env = _env()
    lib = env.lib
    stream = env.stream()
    n = 1 << 18
    x = lib.malloc(4 * n)
    out = lib.malloc(4 * n)
    host = np.full(n, 3.0, np.float32)
    lib.memcpy_h2d_async(x, host.ctypes.data, 4 * n, stream)
    env.synchronize()
    lib.graph_begin_capture(stream)
    tmp = lib.malloc(4 * n + 12345)                         # a size nothing else uses
    lib.scale_f32(tmp, x, n, 2.0, stream)
    lib.scale_f32(out, tmp, n, 5.0, stream)
    lib.free(tmp)
    again = lib.malloc(4 * n + 12345)                       # inside the capture the block may be reused
    assert again == tmp
    lib.free(again)
    handle = ctypes.c_void_p(0)
    lib.graph_end_capture(stream, ctypes.byref(handle))
    outside = lib.malloc(4 * n + 12345)                     # outside it may not
    assert outside != tmp
    for _ in range(2):
        lib.graph_launch(handle.value, stream)
    got = np.empty(n, np.float32)
    lib.memcpy_d2h_async(got.ctypes.data, out, 4 * n, stream)
    env.synchronize()
    assert np.array_equal(got, np.full(n, 30.0, np.float32))
    lib.free(outside)
    lib.graph_destroy(handle.value)
    reserved = lib.pool_reserved_bytes()
    back = [lib.malloc(4 * n + 12345) for _ in range(2)]    # the graph's block and `outside` are both in the pool again
    assert lib.pool_reserved_bytes() == reserved
    for p in back + [x, out]:
        lib.free(p)


def test_tensor_api_runs_without_pytorch_being_imported():
    """The package's CUDA path needs no PyTorch: a fresh interpreter trains a step and never imports it."""
    import os
    import subprocess
    import sys
    import textwrap

    from conftest import ROOT

    code = textwrap.dedent("""
        import sys, numpy as np
        import mytorch_b200 as mt, mytorch_b200.nn.functional as F
        from mytorch_b200.examples.models import ResNet18Cifar
        from mytorch_b200.optim import SGD
        from mytorch_b200.cuda_graph import StepGraph
        mt.manual_seed(1)
        net = ResNet18Cifar((16, 16, 32, 32))
        net.to('cuda:0')
        opt = SGD(net.parameters(), lr=0.05, momentum=0.9)
        rng = np.random.default_rng(0)
        x = mt.tensor(rng.standard_normal((8, 3, 32, 32)).astype(np.float32), device='cuda:0')
        t = mt.tensor(rng.integers(0, 10, 8).astype(np.int64), device='cuda:0')

        def step():
            loss = F.cross_entropy(net(x), t)
            opt.zero_grad()
            loss.backward()
            opt.step()
            return loss

        a = step().item()
        step()
        g = StepGraph(step, [x, t])
        g.capture()
        b = g.replay().item()
        assert np.isfinite(a) and np.isfinite(b) and b < a, (a, b)
        assert 'torch' not in sys.modules, 'PyTorch was imported'
        print('ok')
    """)
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, PYTHONPATH=ROOT))
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
