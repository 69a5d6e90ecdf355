"""Minimal data parallelism: one process per GPU, gradients averaged with one NCCL all-reduce.

The reference has no distributed code at all; this adds the smallest wrapper its training
loop needs to run on 1/2/4/8 GPUs of one box.  The batch is split along dimension 0, every
rank holds a full replica (parameters, momentum buffers, BatchNorm running statistics), and
BatchNorm uses the statistics of the local shard.

On CUDA every parameter owns a window of one flat float32 buffer per bucket, and the backward
kernels (weight gradients, bias gradients, BatchNorm gradients) write ``param.grad`` straight
into that window, so after ``backward`` the buffer is all-reduced in place by NCCL over NVLink
(average) and the multi-tensor SGD kernel reads it in place: no gather or scatter copies.  A
gradient that ended up elsewhere (a parameter used twice accumulates into a fresh tensor) is
copied into its window first.  On the CPU (gloo, used by the tests) gradients are gathered into
the flat buffer pre-scaled by 1/world and summed.  With world size 1 nothing is copied or
communicated.
"""
from __future__ import annotations

import ctypes

import numpy as np

from mytorch_b200.tensor import Tensor


class _DeviceArray:
    """Carrier of the CUDA array interface: lets ``torch.as_tensor`` view pool memory without a copy."""

    def __init__(self, ptr, nelems, typestr):
        self.__cuda_array_interface__ = {"shape": (int(nelems),), "typestr": typestr, "data": (int(ptr), False), "version": 2}


def torch_view(memory, nelems, typestr="<f4"):
    """A PyTorch tensor over a ``CudaMemory`` block (for ``torch.distributed`` only; the block must outlive it)."""
    import torch

    return torch.as_tensor(_DeviceArray(memory.ptr, nelems, typestr), device=f"cuda:{memory.device_index}")


def on_stream(stream_handle, device_index):
    """Context manager that makes a stream of this library PyTorch's current stream, so that a
    collective issued inside is ordered after the work already on that stream."""
    import torch

    return torch.cuda.stream(torch.cuda.ExternalStream(int(stream_handle), device=f"cuda:{device_index}"))


def shard_bounds(n, rank, world):
    """Rows [lo, hi) of a batch of ``n`` rows that belong to ``rank`` (near-equal contiguous shards)."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(array, rank, world):
    lo, hi = shard_bounds(array.shape[0], rank, world)
    return array[lo:hi]


class GradBucket:
    """Offsets of every parameter's gradient inside one flat buffer (256-byte aligned slots)."""

    def __init__(self, params, align_elems=64):
        self.params = list(params)
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            n = int(np.prod(p.shape, dtype=np.int64))
            off += (n + align_elems - 1) // align_elems * align_elems
        self.sizes = [int(np.prod(p.shape, dtype=np.int64)) for p in self.params]
        self.total = max(off, 1)
        self.flat = None      # torch tensor (float32) over the flat buffer, created on first use
        self.flat_mem = None  # CUDA: the pool block behind it

    def _ensure_flat(self):
        if self.flat is None:
            import torch

            dev = self.params[0].device
            if dev.type == "cpu":
                self.flat = torch.zeros(self.total, dtype=torch.float32)
            else:
                from mytorch_b200.backends.cuda.env import CudaEnv, CudaMemory

                env = CudaEnv.instance()
                self.flat_mem = CudaMemory(dev.index, 4 * self.total)
                env.lib.memset_async(self.flat_mem.ptr, 0, 4 * self.total, env.stream())
                self.flat = torch_view(self.flat_mem, self.total)
        return self.flat

    def assign_slots(self):
        """CUDA: give every parameter its window of the flat buffer (``param._grad_slot``); the
        backward operators write the parameter's gradient there (``backends/cuda/ops.py``)."""
        from mytorch_b200.backends.cuda.env import CudaMemoryView

        self._ensure_flat()
        for p, off, n in zip(self.params, self.offsets, self.sizes):
            p._grad_slot = CudaMemoryView(self.flat_mem, 4 * off, 4 * n, self.flat_mem.device_index)

    def pack(self, scale, stream=None):
        """CPU: flat[offset_k : offset_k + n_k] = scale * grad_k for every parameter.  CUDA: the same
        copy (scale 1), but only for gradients that do not already live in their window."""
        flat = self._ensure_flat()
        if self.params[0].device.type == "cpu":
            view = flat.numpy()
            for p, off, n in zip(self.params, self.offsets, self.sizes):
                view[off:off + n] = p.grad._numpy().reshape(-1) * np.float32(scale)
            return flat
        from mytorch_b200.backends.cuda.env import CudaEnv

        stray = [(p, off, n) for p, off, n in zip(self.params, self.offsets, self.sizes)
                 if p.grad._native_array.ptr != p._grad_slot.ptr]
        if stray:
            env = CudaEnv.instance()
            k = len(stray)
            srcs = (ctypes.c_void_p * k)(*[p.grad._native_array.ptr for p, _, _ in stray])
            offs = (ctypes.c_longlong * k)(*[off for _, off, _ in stray])
            sizes = (ctypes.c_longlong * k)(*[n for _, _, n in stray])
            env.lib.pack_scale_f32(k, srcs, offs, sizes, self.flat_mem.ptr, float(scale), env.stream() if stream is None else stream)
        return flat

    def point_grads_at_flat(self):
        """Replace every ``param.grad`` by a tensor that aliases its slot of the flat buffer."""
        flat = self._ensure_flat()
        if self.params[0].device.type == "cpu":
            view = flat.numpy()
            for p, off, n in zip(self.params, self.offsets, self.sizes):
                p.grad = Tensor(cpu_array=view[off:off + n].reshape(p.shape))
            return
        for p in self.params:
            if p.grad._native_array.ptr != p._grad_slot.ptr:  # it was copied into the window by pack()
                g = Tensor(tensor=p.grad)
                g._native_array = p._grad_slot
                p.grad = g


def split_into_buckets(params, count):
    """Split parameters, taken in reverse order of use (the order in which backward finishes
    them), into `count` contiguous groups of roughly equal size in bytes."""
    rev = list(params)[::-1]
    sizes = [int(np.prod(p.shape, dtype=np.int64)) for p in rev]
    total, groups, cur, acc = sum(sizes), [], [], 0
    for p, n in zip(rev, sizes):
        cur.append(p)
        acc += n
        if len(groups) < count - 1 and acc >= total * (len(groups) + 1) / count:
            groups.append(cur)
            cur = []
    if cur:
        groups.append(cur)
    return groups


class DataParallel:
    """Wraps a module; ``reduce_gradients()`` goes between ``loss.backward()`` and ``optimizer.step()``.

    With ``buckets > 1`` the all-reduce of a bucket starts as soon as backward has produced the
    last gradient of that bucket (the deepest layers finish first); on CUDA it runs on a side
    stream, so it overlaps the rest of backward and ``reduce_gradients()`` only waits for it.
    """

    def __init__(self, module, process_group=None, buckets=1):
        import torch.distributed as dist

        self.module = module
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if self.world > 1 else 0
        self.buckets, self._bucket_of, self._remaining, self._events = [], {}, [], []
        self._side, self._on_cuda = None, False
        if self.world > 1:
            params = list(module.parameters())
            on_cuda = params[0].device.type == "cuda"
            groups = split_into_buckets(params, buckets)
            self.buckets = [GradBucket(g) for g in groups]
            self._on_cuda = on_cuda
            if on_cuda:
                for b in self.buckets:
                    b.assign_slots()
            for b, g in enumerate(groups):
                for p in g:
                    self._bucket_of[id(p)] = b
            if len(self.buckets) > 1:
                from mytorch_b200.autograd import DAGTracker

                if on_cuda:
                    from mytorch_b200.backends.cuda.env import CudaEnv

                    self._side = CudaEnv.instance().new_stream()
                DAGTracker.instance().leaf_grad_final_hook = self._on_grad_final
            self._reset()

    def _reset(self):
        self._remaining = [len(b.params) for b in self.buckets]
        self._events = [None] * len(self.buckets)

    def __call__(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def parameters(self):
        return self.module.parameters()

    def shard(self, array):
        return shard_batch(array, self.rank, self.world)

    def _launch_bucket(self, b, stream=None):
        import torch
        import torch.distributed as dist

        bucket = self.buckets[b]
        if not self._on_cuda:
            flat = bucket.pack(1.0 / self.world)
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
            return
        # gradients already sit in the flat buffer; 1/world is an exact scaling for the power-of-two
        # world sizes of one box, so NCCL's average equals the sum of pre-scaled gradients bit for bit
        from mytorch_b200.backends.cuda.env import CudaEnv, Event

        env = CudaEnv.instance()
        index = bucket.params[0].device.index
        env.set_device(index)
        if stream is None:
            flat = bucket.pack(1.0)
            with on_stream(env.stream(), env.current_device()):
                dist.all_reduce(flat, op=dist.ReduceOp.AVG, group=self.group)
            return
        ready = Event()
        ready.record(env.stream())
        env.lib.stream_wait_event(stream, ready.handle)
        weight_gradients = env.side_event()  # weight gradients run on the compute stream's side stream
        if weight_gradients is not None:
            env.lib.stream_wait_event(stream, weight_gradients.handle)
        flat = bucket.pack(1.0, stream=stream)
        with on_stream(stream, env.current_device()):
            dist.all_reduce(flat, op=dist.ReduceOp.AVG, group=self.group)
        done = Event()
        done.record(stream)
        self._events[b] = done

    def _on_grad_final(self, tensor):
        b = self._bucket_of.get(id(tensor))
        if b is None:
            return
        self._remaining[b] -= 1
        if self._remaining[b] == 0:
            self._launch_bucket(b, self._side)

    def reduce_gradients(self):
        if self.world == 1:
            return
        for b, bucket in enumerate(self.buckets):
            if self._remaining[b] > 0:  # not started by the hook (gradients were set by hand, or no hook)
                self._launch_bucket(b, self._side)
        if self._side is not None:
            from mytorch_b200.backends.cuda.env import CudaEnv

            env = CudaEnv.instance()
            for ev in self._events:
                if ev is not None:
                    env.lib.stream_wait_event(env.stream(), ev.handle)
        for bucket in self.buckets:
            bucket.point_grads_at_flat()
        self._reset()

    def broadcast_parameters(self, src=0):
        """Make every replica start from rank ``src``'s parameters and buffers."""
        if self.world == 1:
            return
        import torch
        import torch.distributed as dist

        for t in list(self.module.parameters()) + list(self.module.buffers()):
            if t.device.type == "cpu":
                dist.broadcast(torch.from_numpy(t._numpy()), src=src, group=self.group)
                continue
            from mytorch_b200.backends.cuda.env import CudaEnv

            env = CudaEnv.instance()
            env.set_device(t.device.index)
            nbytes = t._native_array.nbytes
            with on_stream(env.stream(), env.current_device()):
                dist.broadcast(torch_view(t._native_array, nbytes, "|u1"), src=src, group=self.group)
