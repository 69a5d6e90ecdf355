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
    ahead: while the caller computes on batch k, batch k+1 travels host -> page-locked buffer -> device
    staging buffer on a side stream; the compute stream only waits for the copy's event (and converts
    images to the channels-last device layout) when the batch is handed over.  Two sets of buffers
    alternate; a set is refilled only after the compute stream has consumed it.  ``dtypes`` optionally
    casts each element on the host first (labels to int64, as the reference's ``y.to(device, mytorch.int64)``)."""

    def __init__(self, loader, device="cuda:0", dtypes=None):
        self.loader, self.device, self.dtypes = loader, device, dtypes

    def __len__(self):
        return len(self.loader)

    def _stage(self, env, stream, batch, slot):
        from mytorch_b200.backends.cuda.env import CudaMemory, Event, PinnedBuffer

        if slot.get("consumed") is not None:
            slot["consumed"].synchronize()   # host side: the pinned buffers are about to be overwritten
        staged = []
        for k, t in enumerate(batch):
            a = t._numpy()
            if self.dtypes is not None and self.dtypes[k] is not None:
                a = a.astype(self.dtypes[k].np_dtype, copy=False)
            key = (k, a.shape, a.dtype.str)
            bufs = slot.get(key)
            if bufs is None:
                bufs = slot[key] = (PinnedBuffer(a.shape, a.dtype), CudaMemory(None, max(a.nbytes, 1)))
            pinned, raw = bufs
            pinned.array[...] = a
            raw.write_from(pinned.array, stream=stream)
            staged.append((raw, a.shape, a.dtype))
        event = Event()
        event.record(stream)
        return staged, event

    def _hand_over(self, env, staged, event, slot):
        from mytorch_b200.backends.cuda.env import Event
        from mytorch_b200.backends.cuda.ops import _nontrivial_nhwc
        from mytorch_b200.dtype import DType

        env.lib.stream_wait_event(env.stream(), event.handle)
        out = []
        for raw, shape, np_dtype in staged:
            t = Tensor(shape=shape, dtype=DType.from_np_dtype(np_dtype), device=self.device)
            if _nontrivial_nhwc(t):
                n, c, h, w = shape
                env.lib.nchw_to_nhwc_f32(raw.ptr, t._native_array.ptr, n, c, h, w, env.stream())
            else:
                t._native_array.copy_from(raw, t._native_array.nbytes)
            out.append(t)
        slot["consumed"] = Event()
        slot["consumed"].record(env.stream())
        return out

    def __iter__(self):
        from mytorch_b200.backends.cuda.env import CudaEnv
        from mytorch_b200.tensor import Device

        env = CudaEnv.instance()
        env.set_device(Device(self.device).index)
        stream = env.new_stream()
        slots = [{}, {}]
        pending, k = None, 0
        try:
            for batch in self.loader:
                slot = slots[k & 1]
                staged, event = self._stage(env, stream, batch, slot)
                if pending is not None:
                    yield self._hand_over(env, *pending)
                pending, k = (staged, event, slot), k + 1
            if pending is not None:
                yield self._hand_over(env, *pending)
        finally:
            env.lib.stream_synchronize(stream)
            env.lib.stream_destroy(stream)
