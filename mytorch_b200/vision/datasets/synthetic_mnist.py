"""A seeded stand-in with the shape of MNIST (``mytorch/vision/datasets/mnist.py:26-103`` downloads and
parses the real files, which are not available offline): 28x28 uint8 images in ten classes.  Every
class has its own random stroke pattern; a sample is that pattern shifted by up to two pixels with
noise on top, so a small CNN can learn it.  No image of the real dataset is reproduced."""
import numpy as np

from mytorch_b200.utils.data.dataset import Dataset


class SyntheticMNIST(Dataset):
    def __init__(self, count=4096, train=True, transform=None, seed=1000):
        rng = np.random.default_rng(seed)                       # the class patterns are shared by train and test
        coarse = rng.random((10, 7, 7)) < 0.35
        self.patterns = np.kron(coarse, np.ones((4, 4))).astype(np.float32)
        self.rng_seed = seed + (1 if train else 2)
        self.count, self.transform = int(count), transform
        rng = np.random.default_rng(self.rng_seed)
        self.labels = rng.integers(0, 10, self.count)
        self.shifts = rng.integers(-2, 3, (self.count, 2))

    def __len__(self):
        return self.count

    def __getitem__(self, index):
        label = int(self.labels[index])
        noise = np.random.default_rng(self.rng_seed * 1000003 + index).random((28, 28), dtype=np.float32)
        img = np.roll(self.patterns[label], tuple(self.shifts[index]), axis=(0, 1)) * 0.8 + 0.35 * noise
        img = (np.clip(img, 0, 1) * 255).astype(np.uint8)
        return (self.transform(img) if self.transform is not None else img), label
