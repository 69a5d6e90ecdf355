"""Batching over a dataset (``mytorch/utils/data/data_loader.py:10-62``) and a device feed for it.

``DataLoader`` keeps the reference's interface and collate rules: samples are tuples / lists whose
elements are NumPy arrays (stacked along a new first axis), numbers (one 1-D tensor) or CPU tensors
(stacked); it yields lists of CPU tensors.  Like the reference it draws one seed from the global
generator per epoch when ``shuffle`` is set, and like the reference it then walks the dataset in
index order (``data_loader.py:19-25`` builds the permutation but indexes with the loop counter), so
the batches of the two implementations are the same.

``DevicePrefetcher`` plays the role of the blocking ``x.to(device)`` calls of the reference's training
loop (``mytorch/examples/mnist.py:70-73``): batch k+1 is copied from pinned host memory on a side
stream while the model works on batch k.
"""
import numbers

import numpy as np

from mytorch_b200.rand_generator import RandGenerator
from mytorch_b200.tensor import Tensor


class DataLoader:
    def __init__(self, dataset, batch_size=1, shuffle=False):
        self.dataset = dataset
        self.shuffle = shuffle
        self.batch_size = batch_size

    def __len__(self):
        return (len(self.dataset) + self.batch_size - 1) // self.batch_size

    def __iter__(self):
        count = len(self.dataset)
        if self.shuffle:
            RandGenerator.instance().generate()  # consumed exactly as the reference consumes it
        for start in range(0, count, self.batch_size):
            yield self._default_collate([self.dataset[i] for i in range(start, min(start + self.batch_size, count))])

    @staticmethod
    def _default_collate(samples):
        first = samples[0]
        if not isinstance(first, (list, tuple)):
            raise RuntimeError(f"Invalid element type in default collate: {type(first)}")
        batch = []
        for k, element in enumerate(first):
            column = [s[k] for s in samples]
            if isinstance(element, np.ndarray):
                batch.append(Tensor(cpu_array=np.stack(column, axis=0)))
            elif isinstance(element, numbers.Number):
                batch.append(Tensor(cpu_array=np.array(column)))
            elif isinstance(element, Tensor):
                batch.append(Tensor(cpu_array=np.stack([t._numpy() for t in column], axis=0)))
            else:
                raise RuntimeError(f"Invalid data type in default collate: {type(element)}")
        return batch


class DevicePrefetcher:
    """Iterates a loader of CPU-tensor batches and yields the same batches as CUDA tensors, one batch
    ahead: while the caller computes on batch k, batch k+1 travels host -> pinned buffer -> device on a
    side stream; the compute stream only waits for the copy's event (and converts images to the
    channels-last device layout) when the batch is handed over.  ``dtypes`` optionally casts each
    element on the host first (labels to int64, as the reference's ``y.to(device, mytorch.int64)``)."""

    def __init__(self, loader, device="cuda:0", dtypes=None):
        self.loader, self.device, self.dtypes = loader, device, dtypes

    def __len__(self):
        return len(self.loader)

    def _stage(self, env, stream, batch, slot):
        torch = env.torch
        staged = []
        with torch.cuda.stream(stream):
            for k, t in enumerate(batch):
                a = t._numpy()
                if self.dtypes is not None and self.dtypes[k] is not None:
                    a = a.astype(self.dtypes[k].np_dtype, copy=False)
                a = np.ascontiguousarray(a)
                key = (k, a.shape, a.dtype.str)
                pinned = slot.get(key)
                if pinned is None:
                    pinned = slot[key] = torch.empty(a.nbytes, dtype=torch.uint8).pin_memory()
                pinned.numpy()[:] = a.reshape(-1).view(np.uint8)
                raw = env.alloc(a.nbytes)
                raw.copy_(pinned, non_blocking=True)
                raw.record_stream(torch.cuda.current_stream())
                staged.append((raw, a.shape, a.dtype))
            event = torch.cuda.Event()
            event.record(stream)
        return staged, event

    def _hand_over(self, env, staged, event):
        from mytorch_b200.backends.cuda.ops import _nontrivial_nhwc
        from mytorch_b200.dtype import DType

        torch = env.torch
        torch.cuda.current_stream().wait_event(event)
        out = []
        for raw, shape, np_dtype in staged:
            raw.record_stream(torch.cuda.current_stream())
            t = Tensor(shape=shape, dtype=DType.from_np_dtype(np_dtype), device=self.device)
            if _nontrivial_nhwc(t):
                n, c, h, w = shape
                env.lib.nchw_to_nhwc_f32(raw.data_ptr(), t._native_array.ptr, n, c, h, w, env.stream())
            else:
                t._native_array._buf[: raw.numel()].copy_(raw, non_blocking=True)
            out.append(t)
        return out

    def __iter__(self):
        from mytorch_b200.backends.cuda.env import CudaEnv
        from mytorch_b200.tensor import Device

        env = CudaEnv.instance()
        env.set_device(Device(self.device).index)
        stream = env.torch.cuda.Stream()
        slots = [{}, {}]           # pinned host buffers, two sets: one is being filled while the other is in flight
        events = [None, None]
        pending, k = None, 0
        for batch in self.loader:
            if events[k & 1] is not None:
                events[k & 1].synchronize()   # its pinned buffers are about to be overwritten
            staged, event = self._stage(env, stream, batch, slots[k & 1])
            events[k & 1] = event
            if pending is not None:
                yield self._hand_over(env, *pending)
            pending, k = (staged, event), k + 1
        if pending is not None:
            yield self._hand_over(env, *pending)
