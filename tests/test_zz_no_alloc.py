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
    for rows, c, scale in [(4096, 64, 1.0), (777, 24, 0.5), (50000, 512, 1.0), (33, 7, 2.0)]:
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
