"""Whole-step CUDA graph capture and a double-buffered input feed.

A training step issues a few hundred small launches; at 64 images per GPU the host cannot
issue them as fast as a B200 retires them.  ``StepGraph`` runs a step function once under
stream capture (every operator launches on the current stream, allocates from the caching
allocator's graph pool and never synchronises) and afterwards replays it as a single launch.
Inputs are static device tensors refilled from host memory before each replay.

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
        from mytorch_b200.backends.cuda.env import CudaEnv

        self.env = CudaEnv.instance()
        torch = self.env.torch
        self.inputs = list(static_inputs)
        self.copy_stream = torch.cuda.Stream()
        # two staging slots per input, in the logical (host) layout
        self.slots = [[self.env.alloc(t._native_array.nbytes, t.device.index) for _ in range(2)] for t in self.inputs]
        self.copied = [None, None]    # event: slot filled by the copy stream
        self.consumed = [None, None]  # event: slot read by the compute stream
        self.next_slot = 0
        self.staged_slot = None

    def _as_bytes(self, host):
        torch = self.env.torch
        src = host if isinstance(host, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(host))
        return src.reshape(-1).view(torch.uint8)

    def stage(self, host_arrays):
        """Start copying a batch (NumPy arrays or, for truly asynchronous copies, pinned torch CPU
        tensors, in the logical NCHW layout) into the spare slot.  Returns immediately."""
        torch = self.env.torch
        slot = self.next_slot
        with torch.cuda.stream(self.copy_stream):
            if self.consumed[slot] is not None:
                self.copy_stream.wait_event(self.consumed[slot])
            for bufs, host in zip(self.slots, host_arrays):
                src = self._as_bytes(host)
                bufs[slot][: src.numel()].copy_(src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        self.copied[slot] = ev
        self.staged_slot = slot
        self.next_slot = slot ^ 1

    def commit(self):
        """On the compute stream: wait for the staged batch and move it into the static inputs."""
        from mytorch_b200.backends.cuda.ops import _nontrivial_nhwc

        torch = self.env.torch
        slot = self.staged_slot
        if slot is None:
            raise RuntimeError("no batch has been staged")
        stream = torch.cuda.current_stream()
        stream.wait_event(self.copied[slot])
        for t, bufs in zip(self.inputs, self.slots):
            if _nontrivial_nhwc(t):
                n, c, h, w = t.shape
                self.env.lib.nchw_to_nhwc_f32(bufs[slot].data_ptr(), t._native_array.ptr, n, c, h, w, self.env.stream())
            else:
                nbytes = t._native_array.nbytes
                t._native_array._buf[:nbytes].copy_(bufs[slot][:nbytes], non_blocking=True)
        ev = torch.cuda.Event()
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
        import torch

        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.result = self.step_fn()
        torch.cuda.synchronize()
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
        self.graph.replay()
        return self.result
