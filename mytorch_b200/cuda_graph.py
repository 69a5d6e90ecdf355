"""Whole-step CUDA graph capture and a double-buffered input feed.

A training step issues a few hundred small launches; at 64 images per GPU the host cannot
issue them as fast as a B200 retires them.  ``StepGraph`` runs a step function once under
stream capture (every operator launches on the device's compute stream, takes its memory from
the library's pool, whose blocks are then owned by the graph, and never synchronises) and
afterwards replays it as a single launch.  Inputs are static device tensors refilled from host
memory before each replay.

``InputPrefetcher`` plays the role of the reference's blocking ``x.to(device)`` in its training
loop (``mytorch/examples/mnist.py:70-88``, ``mytorch/backends/cuda/env.py:553-561``): the next
batch is copied from pinned host memory on a side stream into a spare staging slot while the
current step runs, and handed to the static input tensors (with the NCHW -> channels-last
conversion for images) on the compute stream just before the next replay.
"""
from __future__ import annotations

import numpy as np


class InputPrefetcher:
    def __init__(self, static_inputs):
        from mytorch_b200.backends.cuda.env import CudaEnv, CudaMemory

        self.env = CudaEnv.instance()
        self.inputs = list(static_inputs)
        self.env.set_device(self.inputs[0].device.index)
        self.copy_stream = self.env.new_stream()
        # two staging slots per input, in the logical (host) layout
        self.slots = [[CudaMemory(t.device.index, t._native_array.nbytes) for _ in range(2)] for t in self.inputs]
        self.copied = [None, None]    # event: slot filled by the copy stream
        self.consumed = [None, None]  # event: slot read by the compute stream
        self.next_slot = 0
        self.staged_slot = None

    def stage(self, host_arrays):
        """Start copying a batch (NumPy arrays or pinned host buffers, in the logical NCHW layout; the
        memory must stay valid until the copy has run, page-locked memory makes it asynchronous) into
        the spare slot.  Returns immediately."""
        from mytorch_b200.backends.cuda.env import Event

        slot = self.next_slot
        if self.consumed[slot] is not None:
            self.env.lib.stream_wait_event(self.copy_stream, self.consumed[slot].handle)
        for bufs, host in zip(self.slots, host_arrays):
            bufs[slot].write_from(host if hasattr(host, "data_ptr") else np.ascontiguousarray(host), stream=self.copy_stream)
        ev = Event()
        ev.record(self.copy_stream)
        self.copied[slot] = ev
        self.staged_slot = slot
        self.next_slot = slot ^ 1

    def commit(self):
        """On the compute stream: wait for the staged batch and move it into the static inputs."""
        from mytorch_b200.backends.cuda.env import Event
        from mytorch_b200.backends.cuda.ops import _nontrivial_nhwc

        slot = self.staged_slot
        if slot is None:
            raise RuntimeError("no batch has been staged")
        stream = self.env.stream()
        self.env.lib.stream_wait_event(stream, self.copied[slot].handle)
        for t, bufs in zip(self.inputs, self.slots):
            if _nontrivial_nhwc(t):
                n, c, h, w = t.shape
                self.env.lib.nchw_to_nhwc_f32(bufs[slot].ptr, t._native_array.ptr, n, c, h, w, stream)
            else:
                t._native_array.copy_from(bufs[slot], t._native_array.nbytes)
        ev = Event()
        ev.record(stream)
        self.consumed[slot] = ev
        self.staged_slot = None


class StepGraph:
    def __init__(self, step_fn, static_inputs=()):
        self.step_fn = step_fn
        self.static_inputs = list(static_inputs)
        self.graph = None
        self.result = None
        self._prefetcher = None

    def capture(self):
        import ctypes

        from mytorch_b200.backends.cuda.env import CudaEnv

        env = CudaEnv.instance()
        if self.static_inputs:
            env.set_device(self.static_inputs[0].device.index)
        stream = env.stream()
        env.synchronize()
        env.lib.graph_begin_capture(stream)
        env._capturing = True
        try:
            self.result = self.step_fn()
        finally:
            env._capturing = False
            handle = ctypes.c_void_p(0)
            env.lib.graph_end_capture(stream, ctypes.byref(handle))
        self.graph = handle.value
        self._env, self._stream = env, stream
        env.synchronize()
        return self.result

    def load_inputs(self, host_arrays):
        from mytorch_b200.backends.cuda.ops import upload_into

        for t, a in zip(self.static_inputs, host_arrays):
            upload_into(t, a)

    def prefetch(self, host_arrays):
        """Begin the host->device copy of the batch for the *next* ``replay(prefetched=True)``."""
        if self._prefetcher is None:
            self._prefetcher = InputPrefetcher(self.static_inputs)
        self._prefetcher.stage(host_arrays)

    def replay(self, host_arrays=None, prefetched=False):
        if prefetched:
            self._prefetcher.commit()
        elif host_arrays is not None:
            self.load_inputs(host_arrays)
        self._env.lib.graph_launch(self.graph, self._stream)
        return self.result

    def destroy(self):
        """Release the executable graph and the pool blocks only it kept alive."""
        if self.graph:
            self._env.synchronize()
            self._env.lib.graph_destroy(self.graph)
            self.graph = None
