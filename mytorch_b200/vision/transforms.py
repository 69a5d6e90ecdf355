"""Image transforms on NumPy arrays (``mytorch/vision/transforms.py:8-44``): ``Compose``, ``ToTensor``
(uint8 HxW or HxWxC -> float32 CxHxW in [0, 1]) and ``Normalize``.  They return NumPy arrays, which
``DataLoader`` stacks into one CPU tensor per batch; nothing is computed on CPU tensors."""
import numpy as np


class Compose:
    def __init__(self, transforms):
        self.transforms = transforms

    def __call__(self, img):
        for t in self.transforms:
            img = t(img)
        return img


class ToTensor:
    def __call__(self, pic):
        data = (np.asarray(pic) / 255.0).astype(np.float32)
        if data.ndim == 2:
            return data[None]
        if data.ndim == 3:
            return np.ascontiguousarray(np.transpose(data, (2, 0, 1)))
        raise NotImplementedError(f"ToTensor expects an HxW or HxWxC image, got shape {data.shape}")


class Normalize:
    def __init__(self, mean, std):
        self.mean, self.std = np.float32(mean), np.float32(std)

    def __call__(self, x):
        return ((x - self.mean) / self.std).astype(np.float32)
