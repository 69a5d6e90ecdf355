"""Whole-step CUDA graph capture.

A training step issues a few hundred small launches; at 64 images per GPU the host cannot
issue them as fast as a B200 retires them.  ``StepGraph`` runs a step function once under
stream capture (every operator launches on the current stream, allocates from the caching
allocator's graph pool and never synchronises) and afterwards replays it as a single launch.
Inputs are static device tensors refilled from host memory before each replay.
"""
from __future__ import annotations


class StepGraph:
    def __init__(self, step_fn, static_inputs=()):
        self.step_fn = step_fn
        self.static_inputs = list(static_inputs)
        self.graph = None
        self.result = None

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

    def replay(self, host_arrays=None):
        if host_arrays is not None:
            self.load_inputs(host_arrays)
        self.graph.replay()
        return self.result
