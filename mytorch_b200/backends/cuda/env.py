"""CUDA runtime glue: the kernel library (ctypes over its C ABI), device memory and streams.

Plays the role of the reference's ``mytorch/backends/cuda/env.py`` (library loader
``:341-393``, ``CudaMemory`` ``:524-561``, ``allocate_memory`` / ``transfer_memory``
``:564-580``).  Device memory, the current stream and host<->device copies come from PyTorch's
CUDA runtime (caching allocator, so repeated steps reuse the same blocks and a whole step can
be captured in a CUDA graph); all arithmetic is done by ``libmytorch_b200.so``.

There is no fallback: if the library is missing or the device is not sm_100, the first CUDA
operation raises.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from mytorch_b200.backends.backend_dispatcher import BackendDispatcher

_P, _I, _L, _F, _D = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_double

_CONV = [_I] * 11
_POOL = [_I] * 10
_SIGNATURES = {
    "mtb_version": ([], _I),
    "mtb_device_check": ([], _I),
    "mtb_fill_f32": ([_P, _L, _F, _P], _I),
    "mtb_copy_f32": ([_P, _P, _L, _P], _I),
    "mtb_scale_f32": ([_P, _P, _L, _F, _P], _I),
    "mtb_relu_forward_f32": ([_P, _P, _L, _P], _I),
    "mtb_relu_backward_f32": ([_P, _P, _P, _L, _P], _I),
    "mtb_add_f32": ([_P, _P, _P, _L, _F, _P], _I),
    "mtb_mul_f32": ([_P, _P, _P, _L, _P], _I),
    "mtb_add_bias_rows_f32": ([_P, _P, _P, _L, _I, _F, _P], _I),
    "mtb_binary_strided_f32": ([_I, _I, _P, _P, _P, _P, _P, _P, _P, _F, _P], _I),
    "mtb_resize_channels_f32": ([_P, _P, _L, _I, _I, _P], _I),
    "mtb_nchw_to_nhwc_f32": ([_P, _P, _I, _I, _I, _I, _P], _I),
    "mtb_nhwc_to_nchw_f32": ([_P, _P, _I, _I, _I, _I, _P], _I),
    "mtb_cast": ([_I, _P, _P, _L, _P], _I),
    "mtb_batch_norm2d_workspace_bytes": ([_I, _I, _I, _I], _L),
    "mtb_batch_norm2d_forward_f32": ([_I, _I, _I, _I, _P, _P, _P, _D, _I, _D, _P, _P, _P, _P, _P, _I, _P, _L, _P], _I),
    "mtb_batch_norm2d_backward_f32": ([_I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _D, _I, _P, _P, _P, _P, _L, _P], _I),
    "mtb_batch_norm2d_add_relu_forward_f32": ([_I, _I, _I, _I, _P, _P, _P, _P, _D, _I, _D, _P, _P, _P, _P, _P, _P, _I, _P, _L, _P], _I),
    "mtb_batch_norm2d_add_relu_backward_f32": ([_I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _D, _P, _P, _P, _P, _P, _L, _P], _I),
    "mtb_add_relu_f32": ([_P, _P, _P, _L, _P], _I),
    "mtb_add_relu_backward_f32": ([_P, _P, _P, _P, _L, _P], _I),
    "mtb_colsum_workspace_bytes": ([_I], _L),
    "mtb_colsum_f32": ([_P, _L, _I, _F, _P, _P, _L, _P], _I),
    "mtb_colsum_noalloc_f32": ([_P, _L, _I, _F, _P, _P], _I),
    "mtb_nhwc_spatial_sum_f32": ([_P, _P, _I, _I, _I, _F, _P], _I),
    "mtb_nhwc_spatial_bcast_f32": ([_P, _P, _I, _I, _I, _F, _P], _I),
    "mtb_sum_strided_f32": ([_P, _P, _I, _P, _P, _I, _P, _P, _F, _P], _I),
    "mtb_max_strided_f32": ([_P, _P, _P, _I, _P, _P, _L, _L, _P], _I),
    "mtb_max_backward_f32": ([_P, _P, _P, _L, _I, _P, _P, _L, _P], _I),
    "mtb_eq_strided": ([_I, _I, _P, _P, _P, _P, _P, _P, _P], _I),
    "mtb_max_pool2d_forward_f32": (_POOL + [_P, _P, _P, _P], _I),
    "mtb_max_pool2d_backward_f32": (_POOL + [_P, _P, _P, _P, _P, _P], _I),
    "mtb_max_pool2d_argmax_u8": ([_P, _P, _L, _P], _I),
    "mtb_cross_entropy_workspace_bytes": ([_I], _L),
    "mtb_cross_entropy_forward_f32": ([_I, _I, _P, _P, _P, _P, _L, _P], _I),
    "mtb_cross_entropy_backward_f32": ([_I, _I, _P, _P, _P, _P, _P], _I),
    "mtb_sgd_f32": ([_P, _P, _P, _L, _I, _D, _D, _D, _D, _I, _I, _D, _P], _I),
    "mtb_sgd_multi_f32": ([_I, _P, _P, _P, _P, _P, _D, _D, _D, _D, _I, _I, _D, _P], _I),
    "mtb_pack_scale_f32": ([_I, _P, _P, _P, _P, _D, _P], _I),
    "mtb_conv2d_workspace_bytes": (_CONV, _L),
    "mtb_conv2d_plan_f32": (_CONV + [_P], _I),
    "mtb_conv2d_forward_f32": (_CONV + [_P, _P, _P, _P, _I, _P], _I),
    "mtb_conv2d_stats_max_rows": ([], _I),
    "mtb_conv2d_forward_stats_f32": (_CONV + [_P, _P, _P, _P, _I, _P, _P, _P], _I),
    "mtb_batch_norm2d_forward_prestats_f32": ([_I, _I, _I, _I, _P, _P, _P, _D, _D, _P, _P, _P, _P, _P, _I, _P, _I, _P, _L, _P], _I),
    "mtb_conv2d_dgrad_f32": (_CONV + [_P, _P, _P, _P, _L, _P], _I),
    "mtb_conv2d_dgrad_add_f32": (_CONV + [_P, _P, _P, _P, _P, _L, _P], _I),
    "mtb_conv2d_wgrad_f32": (_CONV + [_P, _P, _P, _P, _L, _P], _I),
    "mtb_gemm_f32": ([_I, _I, _I, _P, _I, _P, _I, _P, _I, _P, _P], _I),
    "mtb_tc_status": ([_P], _I),
    "mtb_tc_wait_selftest": ([_L, _I, _P], _I),
}

LIBRARY_PATH = os.environ.get(
    "MYTORCH_B200_LIB",
    os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "lib", "libmytorch_b200.so"),
)


class NativeError(RuntimeError):
    pass


class NativeLibrary:
    """ctypes view of ``libmytorch_b200.so``; every wrapped call raises on a non-zero status."""

    def __init__(self, path=LIBRARY_PATH):
        if not os.path.exists(path):
            raise NativeError(
                f"kernel library not found at {path}; build it with `python -m mytorch_b200.build` "
                "(there is no fallback implementation)")
        self._dll = ctypes.CDLL(path)
        self._dll.mtb_last_error.restype = ctypes.c_char_p
        self._dll.mtb_last_error.argtypes = []
        self.launches = 0
        for name, (argtypes, restype) in _SIGNATURES.items():
            fn = getattr(self._dll, name)
            fn.argtypes = argtypes
            fn.restype = restype
            setattr(self, name[4:], self._checked(name, fn) if restype is _I and name not in ("mtb_version", "mtb_conv2d_stats_max_rows") else fn)

    def _checked(self, name, fn):
        def call(*args):
            rc = fn(*args)
            if rc != 0:
                raise NativeError(f"{name} failed ({rc}): {self._dll.mtb_last_error().decode()}")
            self.launches += 1
            return rc

        return call

    def exported(self, name):
        return hasattr(self._dll, name)


class CudaEnv:
    """Per-process CUDA state: the library, and one grow-only scratch buffer per device."""

    _instance = None

    @classmethod
    def instance(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def __init__(self):
        import torch

        if not torch.cuda.is_available():
            raise NativeError("no CUDA device is available; the cuda backend has no CPU fallback")
        self.torch = torch
        self.lib = NativeLibrary()
        self.lib.device_check()
        self._scratch = {}
        self._retired_scratch = []

    def stream(self):
        return self.torch.cuda.current_stream().cuda_stream

    def capturing(self):
        return bool(self.torch.cuda.is_current_stream_capturing())

    def tensor_core_status(self):
        """Synchronises and returns the status word of the tensor-core kernels (0 = fine; non-zero
        = a bounded wait inside a kernel ran out and the kernel gave up).  Reading clears it."""
        out = ctypes.c_int(0)
        self.lib.tc_status(ctypes.byref(out))
        return out.value

    def set_device(self, index):
        if index is not None and index != self.torch.cuda.current_device():
            self.torch.cuda.set_device(index)

    def alloc(self, nbytes, index=None):
        dev = self.torch.cuda.current_device() if index is None else index
        return self.torch.empty((max(int(nbytes), 1),), dtype=self.torch.uint8, device=f"cuda:{dev}")

    def workspace(self, nbytes):
        """Scratch for kernels that need it (split-K partials, per-CTA reduction partials).
        One buffer per device, shared by all operators: they run in order on one stream."""
        dev = self.torch.cuda.current_device()
        buf = self._scratch.get(dev)
        if buf is None or buf.numel() < nbytes:
            if buf is not None:
                # a captured graph may hold this block's address: it is kept for the life of the
                # process so that the allocator can never hand it to a tensor a replay would overwrite
                self._retired_scratch.append(buf)
            buf = self.alloc(max(int(nbytes), 1 << 20), dev)
            self._scratch[dev] = buf
        return buf.data_ptr(), buf.numel()


class CudaMemory:
    """A device allocation. ``ptr`` is the raw device address; ``read`` / ``write`` move bytes
    between it and NumPy arrays without interpreting any layout."""

    def __init__(self, device_index, nbytes):
        env = CudaEnv.instance()
        self.device_index = env.torch.cuda.current_device() if device_index is None else device_index
        self.nbytes = int(nbytes)
        self._buf = env.alloc(self.nbytes, self.device_index)
        self.ptr = self._buf.data_ptr()

    def read(self, shape, np_dtype):
        torch = CudaEnv.instance().torch
        n = int(np.prod(shape, dtype=np.int64)) * np.dtype(np_dtype).itemsize
        host = self._buf[:n].cpu().numpy()
        return host.view(np_dtype).reshape(shape).copy()

    def write(self, array, non_blocking=False):
        torch = CudaEnv.instance().torch
        a = np.ascontiguousarray(array)
        src = torch.from_numpy(a.reshape(-1).view(np.uint8))
        self._buf[: src.numel()].copy_(src, non_blocking=non_blocking)

    def write_from(self, host_tensor, non_blocking=True):
        """Copy from a (pinned) torch host tensor of bytes."""
        self._buf[: host_tensor.numel()].copy_(host_tensor, non_blocking=non_blocking)

    def destroy(self):
        self._buf = None
        self.ptr = 0


@BackendDispatcher.instance().register_backend_function("cuda", "allocate_memory")
def cuda_allocate_memory(device_index, nbytes):
    return CudaMemory(device_index, nbytes)


@BackendDispatcher.instance().register_backend_function("cuda", "transfer_memory")
def cuda_transfer_memory(dst, src):
    dst._buf[: src.nbytes].copy_(src._buf[: src.nbytes])


class CudaMemoryView(CudaMemory):
    """A window into another allocation (used for gradient tensors that live inside one flat
    all-reduce buffer). Keeps the parent buffer alive."""

    def __init__(self, torch_bytes_slice, device_index):
        self.device_index = device_index
        self.nbytes = int(torch_bytes_slice.numel())
        self._buf = torch_bytes_slice
        self.ptr = torch_bytes_slice.data_ptr()
