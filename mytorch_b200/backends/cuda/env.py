"""CUDA runtime glue: the kernel library (ctypes over its C ABI), device memory, streams, events.

Plays the role of the reference's ``mytorch/backends/cuda/env.py`` (library loader
``:341-393``, ``CudaMemory`` ``:524-561``, ``allocate_memory`` / ``transfer_memory``
``:564-580``) and ``memory_allocator.py:16-51``.  Everything comes from ``libmytorch_b200.so``:
the arithmetic kernels and the runtime around them (a size-keyed device memory pool whose blocks
keep their addresses from step to step, asynchronous copies, one compute stream per device,
events, whole-step graph capture).  This module imports neither PyTorch nor any other CUDA
binding; ``mytorch_b200.parallel`` alone uses ``torch.distributed`` for the NCCL all-reduce.

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
    "mtb_conv2d_forward_f32": (_CONV + [_P, _P, _P, _P, _I, _P, _L, _P], _I),
    "mtb_conv2d_stats_max_rows": ([], _I),
    "mtb_conv2d_forward_stats_f32": (_CONV + [_P, _P, _P, _P, _I, _P, _P, _P, _L, _P], _I),
    "mtb_batch_norm2d_forward_prestats_f32": ([_I, _I, _I, _I, _P, _P, _P, _D, _D, _P, _P, _P, _P, _P, _I, _P, _I, _P, _L, _P], _I),
    "mtb_conv2d_dgrad_f32": (_CONV + [_P, _P, _P, _P, _L, _P], _I),
    "mtb_conv2d_dgrad_add_f32": (_CONV + [_P, _P, _P, _P, _P, _L, _P], _I),
    "mtb_conv2d_dgrad_accumulates_in_place": (_CONV + [_P, _P, _P], _I),
    "mtb_conv2d_wgrad_f32": (_CONV + [_P, _P, _P, _P, _L, _P], _I),
    "mtb_gemm_f32": ([_I, _I, _I, _P, _I, _P, _I, _P, _I, _P, _P], _I),
    "mtb_tc_status": ([_P], _I),
    # runtime
    "mtb_malloc": ([_L], _P),
    "mtb_free": ([_P], _I),
    "mtb_pool_reserved_bytes": ([], _L),
    "mtb_pool_in_use_bytes": ([], _L),
    "mtb_pool_trim": ([], _I),
    "mtb_set_device": ([_I], _I),
    "mtb_get_device": ([_P], _I),
    "mtb_device_count": ([_P], _I),
    "mtb_device_synchronize": ([], _I),
    "mtb_mem_get_info": ([_P, _P], _I),
    "mtb_memcpy_h2d_async": ([_P, _P, _L, _P], _I),
    "mtb_memcpy_d2h_async": ([_P, _P, _L, _P], _I),
    "mtb_memcpy_d2d_async": ([_P, _P, _L, _P], _I),
    "mtb_memset_async": ([_P, _I, _L, _P], _I),
    "mtb_host_alloc_pinned": ([_L], _P),
    "mtb_host_free_pinned": ([_P], _I),
    "mtb_stream_create": ([], _P),
    "mtb_stream_destroy": ([_P], _I),
    "mtb_stream_synchronize": ([_P], _I),
    "mtb_stream_wait_event": ([_P, _P], _I),
    "mtb_event_create": ([_I], _P),
    "mtb_event_destroy": ([_P], _I),
    "mtb_event_record": ([_P, _P], _I),
    "mtb_event_synchronize": ([_P], _I),
    "mtb_event_elapsed_ms": ([_P, _P, _P], _I),
    "mtb_graph_begin_capture": ([_P], _I),
    "mtb_graph_end_capture": ([_P, _P], _I),
    "mtb_graph_launch": ([_P, _P], _I),
    "mtb_graph_destroy": ([_P], _I),
    "mtb_tc_wait_selftest": ([_L, _I, _P], _I),
}

LIBRARY_PATH = os.environ.get(
    "MYTORCH_B200_LIB",
    os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "lib", "libmytorch_b200.so"),
)

# entry points that only enqueue or bookkeep: not counted as kernel launches
_NOT_LAUNCHES = {"mtb_free", "mtb_pool_trim", "mtb_set_device", "mtb_get_device", "mtb_device_count", "mtb_device_synchronize", "mtb_mem_get_info",
                 "mtb_memcpy_h2d_async", "mtb_memcpy_d2h_async", "mtb_memcpy_d2d_async", "mtb_memset_async", "mtb_host_free_pinned",
                 "mtb_stream_destroy", "mtb_stream_synchronize", "mtb_stream_wait_event", "mtb_event_destroy", "mtb_event_record",
                 "mtb_event_synchronize", "mtb_event_elapsed_ms", "mtb_graph_begin_capture", "mtb_graph_end_capture", "mtb_graph_launch",
                 "mtb_graph_destroy", "mtb_tc_status", "mtb_device_check", "mtb_conv2d_plan_f32"}


class NativeError(RuntimeError):
    pass


class NativeLibrary:
    """ctypes view of ``libmytorch_b200.so``; every wrapped call raises on a non-zero status (or a
    NULL pointer from the entry points that return one)."""

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
            if restype is _P:
                wrapped = self._pointer(name, fn)
            elif restype is _I and name not in ("mtb_version", "mtb_conv2d_stats_max_rows", "mtb_conv2d_dgrad_accumulates_in_place"):
                wrapped = self._checked(name, fn, name not in _NOT_LAUNCHES)
            else:
                wrapped = fn
            setattr(self, name[4:], wrapped)

    def _checked(self, name, fn, counts):
        def call(*args):
            rc = fn(*args)
            if rc != 0:
                raise NativeError(f"{name} failed ({rc}): {self._dll.mtb_last_error().decode()}")
            if counts:
                self.launches += 1
            return rc

        return call

    def _pointer(self, name, fn):
        def call(*args):
            p = fn(*args)
            if not p:
                raise NativeError(f"{name} failed: {self._dll.mtb_last_error().decode()}")
            return p

        return call

    def exported(self, name):
        return hasattr(self._dll, name)


class Event:
    """A CUDA event (``timing=True`` to measure elapsed time between two of them)."""

    def __init__(self, timing=False):
        self._lib = CudaEnv.instance().lib
        self.handle = self._lib.event_create(int(bool(timing)))

    def record(self, stream=None):
        self._lib.event_record(self.handle, CudaEnv.instance().stream() if stream is None else stream)

    def synchronize(self):
        self._lib.event_synchronize(self.handle)

    def elapsed_ms(self, later):
        ms = ctypes.c_float(0)
        self._lib.event_elapsed_ms(self.handle, later.handle, ctypes.byref(ms))
        return ms.value

    def __del__(self):
        try:
            self._lib.event_destroy(self.handle)
        except Exception:
            pass


class PinnedBuffer:
    """Page-locked host memory, viewed as a NumPy array: copies from it to the device are asynchronous."""

    def __init__(self, shape, np_dtype):
        self._lib = CudaEnv.instance().lib
        self.nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(np_dtype).itemsize
        self.ptr = self._lib.host_alloc_pinned(self.nbytes)
        raw = (ctypes.c_ubyte * max(self.nbytes, 1)).from_address(self.ptr)
        self.array = np.frombuffer(raw, dtype=np_dtype, count=int(np.prod(shape, dtype=np.int64))).reshape(shape)

    def __del__(self):
        try:
            self.array = None
            self._lib.host_free_pinned(self.ptr)
        except Exception:
            pass


class CudaEnv:
    """Per-process CUDA state: the library, one compute stream and one grow-only scratch buffer per device."""

    _instance = None

    @classmethod
    def instance(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def __init__(self):
        self.lib = NativeLibrary()
        count = ctypes.c_int(0)
        try:
            self.lib.device_count(ctypes.byref(count))
        except NativeError as e:
            raise NativeError(f"no CUDA device is available; the cuda backend has no CPU fallback ({e})") from None
        if count.value == 0:
            raise NativeError("no CUDA device is available; the cuda backend has no CPU fallback")
        self.lib.device_check()
        self._streams = {}
        self._scratch = {}
        self._retired_scratch = []
        self._capturing = False
        # weight gradients run beside the rest of backward on a second stream (see fork_side / join_side)
        self._side_streams = {}
        self._side_scratch = {}
        self._side_keepalive = []
        self._side_busy = set()
        self.overlap_weight_gradients = not os.environ.get("MTB_SERIAL_WGRAD")
        from mytorch_b200.autograd import DAGTracker

        DAGTracker.instance().join_hook = self.join_side

    # ---- devices, streams
    def current_device(self):
        dev = ctypes.c_int(0)
        self.lib.get_device(ctypes.byref(dev))
        return dev.value

    def set_device(self, index):
        if index is not None and index != self.current_device():
            self.lib.set_device(int(index))

    def stream(self):
        """The compute stream of the current device: every operator enqueues its work there."""
        dev = self.current_device()
        s = self._streams.get(dev)
        if s is None:
            s = self._streams[dev] = self.lib.stream_create()
        return s

    def new_stream(self):
        return self.lib.stream_create()

    def synchronize(self):
        self.lib.device_synchronize()

    def capturing(self):
        return self._capturing

    def mem_get_info(self):
        free, total = ctypes.c_longlong(0), ctypes.c_longlong(0)
        self.lib.mem_get_info(ctypes.byref(free), ctypes.byref(total))
        return free.value, total.value

    def tensor_core_status(self):
        """Synchronises and returns the status word of the tensor-core kernels (0 = fine; non-zero
        = a bounded wait inside a kernel ran out and the kernel gave up).  Reading clears it."""
        out = ctypes.c_int(0)
        self.lib.tc_status(ctypes.byref(out))
        return out.value

    # ---- a second stream for work nothing on the compute stream waits for until backward ends
    def fork_side(self, keepalive=()):
        """The side stream of the current device, ordered after everything enqueued on the compute
        stream so far.  ``keepalive``: objects whose device memory the side-stream work reads or writes;
        they are held until ``join_side`` so that the pool cannot hand their blocks to compute-stream
        work while the side stream still uses them."""
        dev = self.current_device()
        side = self._side_streams.get(dev)
        if side is None:
            side = self._side_streams[dev] = self.lib.stream_create()
        ev = Event()
        ev.record(self.stream())
        self.lib.stream_wait_event(side, ev.handle)
        self._side_keepalive.extend(keepalive)
        self._side_busy.add(dev)
        return side

    def side_event(self):
        """An event after everything enqueued so far on the current device's side stream (None if idle):
        a third stream that consumes side-stream results (the gradient all-reduce) waits on it directly,
        without making the compute stream wait."""
        dev = self.current_device()
        if dev not in self._side_busy:
            return None
        ev = Event()
        ev.record(self._side_streams[dev])
        return ev

    def join_side(self):
        """Make the compute stream of every device wait for its side stream; release the kept objects."""
        if not self._side_busy:
            return
        current = self.current_device()
        for dev in list(self._side_busy):
            self.set_device(dev)
            ev = Event()
            ev.record(self._side_streams[dev])
            self.lib.stream_wait_event(self.stream(), ev.handle)
        self.set_device(current)
        self._side_busy.clear()
        self._side_keepalive.clear()

    def side_workspace(self, nbytes):
        """Scratch for side-stream kernels (the compute stream's scratch may be in use at the same time)."""
        return self._grow_scratch(self._side_scratch, nbytes)

    # ---- memory
    def workspace(self, nbytes):
        """Scratch for kernels that need it (split-K partials, per-CTA reduction partials).
        One buffer per device, shared by all operators: they run in order on one stream."""
        return self._grow_scratch(self._scratch, nbytes)

    def _grow_scratch(self, table, nbytes):
        dev = self.current_device()
        buf = table.get(dev)
        if buf is None or buf.nbytes < nbytes:
            if buf is not None:
                # a captured graph may hold this block's address: it is kept for the life of the
                # process so that the pool can never hand it to a tensor a replay would overwrite
                self._retired_scratch.append(buf)
            buf = CudaMemory(dev, max(int(nbytes), 1 << 20))
            table[dev] = buf
        return buf.ptr, buf.nbytes


class CudaMemory:
    """A device allocation from the library's pool. ``ptr`` is the raw device address; ``read`` /
    ``write`` move bytes between it and NumPy arrays without interpreting any layout."""

    def __init__(self, device_index, nbytes):
        env = CudaEnv.instance()
        self.device_index = env.current_device() if device_index is None else device_index
        env.set_device(self.device_index)
        self.nbytes = int(nbytes)
        self._lib = env.lib
        self.ptr = env.lib.malloc(max(self.nbytes, 1))

    def read(self, shape, np_dtype):
        env = CudaEnv.instance()
        env.join_side()  # a host read must see what the side stream has produced, too
        env.set_device(self.device_index)
        out = np.empty(shape, dtype=np_dtype)
        env.lib.memcpy_d2h_async(out.ctypes.data, self.ptr, out.nbytes, env.stream())
        env.lib.stream_synchronize(env.stream())
        return out

    def write(self, array):
        """Copy a NumPy array in (pageable memory: the call returns once the bytes are staged)."""
        env = CudaEnv.instance()
        env.set_device(self.device_index)
        a = np.ascontiguousarray(array)
        env.lib.memcpy_h2d_async(self.ptr, a.ctypes.data, a.nbytes, env.stream())
        env.lib.stream_synchronize(env.stream())

    def write_from(self, host, stream=None):
        """Asynchronous copy from host memory that stays valid until the copy has run: a NumPy array
        (page-locked, e.g. ``PinnedBuffer.array``, for a truly asynchronous copy) or any object with
        ``data_ptr()`` / ``numel()`` / ``element_size()`` (a pinned PyTorch CPU tensor)."""
        env = CudaEnv.instance()
        env.set_device(self.device_index)
        src, nbytes = host_pointer(host)
        env.lib.memcpy_h2d_async(self.ptr, src, min(nbytes, self.nbytes), env.stream() if stream is None else stream)

    def copy_from(self, other, nbytes=None):
        env = CudaEnv.instance()
        env.set_device(self.device_index)
        env.lib.memcpy_d2d_async(self.ptr, other.ptr, self.nbytes if nbytes is None else nbytes, env.stream())

    def destroy(self):
        if self.ptr:
            self._lib.free(self.ptr)
            self.ptr = 0

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def host_pointer(host):
    """(address, bytes) of a contiguous host buffer: NumPy array or an object with ``data_ptr()``."""
    if hasattr(host, "data_ptr"):
        return host.data_ptr(), host.numel() * host.element_size()
    if not host.flags["C_CONTIGUOUS"]:
        raise ValueError("host buffer must be contiguous")
    return host.ctypes.data, host.nbytes


@BackendDispatcher.instance().register_backend_function("cuda", "allocate_memory")
def cuda_allocate_memory(device_index, nbytes):
    return CudaMemory(device_index, nbytes)


@BackendDispatcher.instance().register_backend_function("cuda", "transfer_memory")
def cuda_transfer_memory(dst, src):
    dst.copy_from(src, src.nbytes)


class CudaMemoryView(CudaMemory):
    """A window into another allocation (used for gradient tensors that live inside one flat
    all-reduce buffer). Keeps the parent alive; frees nothing."""

    def __init__(self, parent, offset_bytes, nbytes, device_index):
        self.device_index = device_index
        self.nbytes = int(nbytes)
        self._parent = parent
        self.ptr = parent.ptr + int(offset_bytes)

    def destroy(self):
        self.ptr = 0
