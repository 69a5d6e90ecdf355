"""The allocation-free column sum (``mtb_colsum_noalloc_f32``) against the regular entry point.

It exists for callers that can neither supply a scratch buffer nor allocate one (an embedding
runtime whose own arena holds all device memory; a step loop that must not touch the driver's
allocator).  Its scratch is a fixed array inside the library, shared by every call, so the test
makes two calls in a row with different shapes and checks both results, and checks that a
shape beyond the built-in limit is refused with an error instead of overrunning the array.

This file is named to be collected last: a run that stops at the first failure has then
already exercised everything else.
"""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu


def test_noalloc_colsum_matches_workspace_variant_on_consecutive_calls():
    import gpu_util as g
    from mytorch_b200.backends.cuda.env import CudaEnv, NativeError

    env = CudaEnv.instance()
    lib = env.lib
    rng = np.random.default_rng(2024)
    # the last two sit at the limit (1024 channels) and just under it (1023: not a multiple of 4, so the
    # scalar kernel runs over several column blocks)
    for rows, c, scale in [(4096, 64, 1.0), (777, 24, 0.5), (50000, 512, 1.0), (33, 7, 2.0), (3000, 1024, 1.0), (2100, 1023, 0.25)]:
        a = rng.standard_normal((rows, c)).astype(np.float32)
        at = g.dev(a)
        ref_out, new_out = g.dev(np.zeros(c, np.float32)), g.dev(np.full(c, 7.0, np.float32))
        ws, ws_bytes = env.workspace(lib.colsum_workspace_bytes(c))
        lib.colsum_f32(at._native_array.ptr, rows, c, scale, ref_out._native_array.ptr, ws, ws_bytes, env.stream())
        lib.colsum_noalloc_f32(at._native_array.ptr, rows, c, scale, new_out._native_array.ptr, env.stream())
        want = g.host(ref_out)
        got = g.host(new_out)
        assert rel_err(got, want) < 1e-5, (rows, c)
        assert rel_err(got, a.astype(np.float64).sum(axis=0) * scale) < 1e-5, (rows, c)
    with pytest.raises(NativeError, match="exceed the built-in scratch"):
        big = g.dev(np.zeros((8, 2048), np.float32))
        out = g.dev(np.zeros(2048, np.float32))
        lib.colsum_noalloc_f32(big._native_array.ptr, 8, 2048, 1.0, out._native_array.ptr, env.stream())


def test_noalloc_colsum_leaves_free_device_memory_unchanged():
    """After one warm-up call (which may make the driver load the library's device code), further
    calls neither take nor return device memory: the free-memory figure the driver reports stays put."""
    import gpu_util as g
    from mytorch_b200.backends.cuda.env import CudaEnv

    env = CudaEnv.instance()
    rng = np.random.default_rng(7)
    a = rng.standard_normal((20000, 256)).astype(np.float32)
    at, out = g.dev(a), g.dev(np.zeros(256, np.float32))
    call = lambda: env.lib.colsum_noalloc_f32(at._native_array.ptr, 20000, 256, 1.0, out._native_array.ptr, env.stream())
    call()
    env.synchronize()
    free_before, _ = env.mem_get_info()
    pool_before = env.lib.pool_reserved_bytes()
    for _ in range(5):
        call()
    env.synchronize()
    free_after, _ = env.mem_get_info()
    assert env.lib.pool_reserved_bytes() == pool_before
    assert free_after == free_before
    assert rel_err(g.host(out), a.astype(np.float64).sum(axis=0)) < 1e-5
