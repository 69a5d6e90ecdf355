"""DataLoader (collate rules of ``mytorch/utils/data/data_loader.py:28-62``), the image transforms, the
synthetic MNIST-shaped dataset, and on the GPU the double-buffered device feed and the MNIST example
loop (train, evaluate with max / eq / cast / mean, save a checkpoint, resume from it)."""
import numpy as np
import pytest

import mytorch_b200 as mt
from mytorch_b200.utils.data import DataLoader, Dataset, DevicePrefetcher
from mytorch_b200.vision import transforms
from mytorch_b200.vision.datasets import SyntheticMNIST


class _Pairs(Dataset):
    def __init__(self, n):
        self.n = n

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        return np.full((2, 3), i, np.float32), i, mt.tensor(np.array([i, -i], np.float32))


def test_loader_batches_and_collates_like_the_reference():
    loader = DataLoader(_Pairs(10), batch_size=4)
    batches = list(loader)
    assert len(loader) == 3 and [b[0].shape for b in batches] == [(4, 2, 3), (4, 2, 3), (2, 2, 3)]
    assert batches[1][1].dtype is mt.int64 and np.array_equal(batches[1][1]._numpy(), [4, 5, 6, 7])
    assert np.array_equal(batches[2][2]._numpy(), [[8, -8], [9, -9]])
    with pytest.raises(RuntimeError):
        DataLoader._default_collate([5, 6])
    with pytest.raises(RuntimeError):
        DataLoader._default_collate([("a",), ("b",)])


def test_shuffle_draws_one_seed_per_epoch_and_keeps_the_reference_order():
    from mytorch_b200.rand_generator import RandGenerator

    mt.manual_seed(9)
    expected_next = None
    loader = DataLoader(_Pairs(6), batch_size=2, shuffle=True)
    first = [b[1]._numpy().tolist() for b in loader]
    after_one_epoch = RandGenerator.instance().generate()
    mt.manual_seed(9)
    RandGenerator.instance().generate()
    assert RandGenerator.instance().generate() == after_one_epoch
    assert first == [[0, 1], [2, 3], [4, 5]]


def test_transforms_and_synthetic_dataset():
    tf = transforms.Compose([transforms.ToTensor(), transforms.Normalize(0.5, 0.25)])
    img = np.arange(12, dtype=np.uint8).reshape(3, 4)
    out = tf(img)
    assert out.shape == (1, 3, 4) and out.dtype == np.float32 and np.allclose(out, (img[None] / 255.0 - 0.5) / 0.25)
    assert transforms.ToTensor()(np.zeros((5, 6, 3), np.uint8)).shape == (3, 5, 6)
    train, again, test = SyntheticMNIST(64, True, tf), SyntheticMNIST(64, True, tf), SyntheticMNIST(64, False, tf)
    x, y = train[3]
    assert x.shape == (1, 28, 28) and 0 <= y < 10 and np.array_equal(x, again[3][0]) and y == again[3][1]
    assert not np.array_equal(x, test[3][0])
    assert np.array_equal(train.patterns, test.patterns)


@pytest.mark.gpu
def test_device_prefetcher_delivers_every_batch_intact():
    import gpu_util as g

    ds = SyntheticMNIST(200, True, transforms.ToTensor())
    loader = DataLoader(ds, batch_size=48)
    want = list(loader)
    got = list(DevicePrefetcher(loader, g.DEV, dtypes=[None, mt.int64]))
    assert len(got) == len(want) == 5
    for (x, y), (hx, hy) in zip(got, want):
        assert x.device.type == "cuda" and y.dtype is mt.int64
        assert np.array_equal(g.host(x), hx._numpy()) and np.array_equal(g.host(y), hy._numpy())


@pytest.mark.gpu
def test_mnist_example_learns_saves_and_resumes(tmp_path):
    from mytorch_b200.examples.mnist import train_mnist

    mt.manual_seed(1000)
    path = str(tmp_path / "mnist.pt")
    lines = []
    history = train_mnist("cuda:0", epochs=1, train_size=2048, test_size=512, save_ckpt=path, log=lines.append)
    assert history[-1] > 0.9, (history, lines[-3:])
    resumed = train_mnist("cuda:0", epochs=1, train_size=1024, test_size=512, ckpt=path, log=lines.append)
    assert resumed[-1] >= history[-1] - 0.05
    assert any(line.startswith("Accuracy:") for line in lines) and any("Epoch #1" in line for line in lines)
