"""The reference's MNIST example (``mytorch/examples/mnist.py:12-112``) on a synthetic MNIST-shaped
dataset: the same CNN (three Conv-BatchNorm-ReLU-MaxPool stages, two Linear layers), SGD lr 0.1,
batches of 64, accuracy through ``max(dim=1)`` / ``eq`` / cast / ``mean`` exactly as the reference
prints it, checkpoint save / resume in the reference's file format.  Batches reach the GPU through
``DevicePrefetcher`` (copy of batch k+1 overlapped with the step on batch k).

    python -m mytorch_b200.examples.mnist [--device cuda:0] [--epochs 1] [--train-size 4096] [--save-ckpt path] [--ckpt path]
"""
import argparse

import mytorch_b200 as mytorch
import mytorch_b200.nn as nn
import mytorch_b200.nn.functional as F
import mytorch_b200.optim as optim
import mytorch_b200.vision.transforms as transforms
from mytorch_b200.utils.data import DataLoader, DevicePrefetcher
from mytorch_b200.vision.datasets import SyntheticMNIST


class CNN(nn.Module):
    def __init__(self):
        super().__init__()
        self.layer1 = nn.Sequential(
            nn.Conv2d(1, 32, kernel_size=3, padding=1), nn.BatchNorm2d(32), nn.ReLU(), nn.MaxPool2d(2, 2),
            nn.Conv2d(32, 128, kernel_size=3, padding=1), nn.BatchNorm2d(128), nn.ReLU(), nn.MaxPool2d(2, 2),
            nn.Conv2d(128, 32, kernel_size=3, padding=1), nn.BatchNorm2d(32), nn.ReLU(), nn.MaxPool2d(2, 2),
        )
        self.layer2 = nn.Sequential(nn.Linear(32 * 3 * 3, 128), nn.ReLU(), nn.Linear(128, 10))

    def forward(self, x):
        return self.layer2(self.layer1(x).reshape((x.shape[0], -1)))


def get_transform():
    return transforms.Compose([transforms.ToTensor(), transforms.Normalize(0.1307, 0.3081)])


def accuracy_of(logits, target):
    return logits.max(dim=1)[1].eq(target).to(dtype=mytorch.float32)


def train_mnist(device="cuda:0", epochs=1, train_size=4096, test_size=1024, ckpt=None, save_ckpt=None, log=print):
    transform = get_transform()
    train_loader = DataLoader(SyntheticMNIST(train_size, True, transform), batch_size=64, shuffle=True)
    test_loader = DataLoader(SyntheticMNIST(test_size, False, transform), batch_size=64, shuffle=False)
    feed = lambda loader: DevicePrefetcher(loader, device, dtypes=[None, mytorch.int64])

    model = CNN()
    model.to(device)
    optimizer = optim.SGD(model.parameters(), lr=1e-1)
    last_epoch = -1
    if ckpt is not None:
        state = mytorch.load(ckpt, map_location=device)
        optimizer.load_state_dict(state["optimizer"])
        model.load_state_dict(state["model"])
        last_epoch = state["epoch"]
        log(f"Accuracy: {state['accuracy'] * 100:.2f}%")

    history = []
    for epoch in range(last_epoch + 1, last_epoch + 1 + epochs):
        model.train()
        for i, (x, target) in enumerate(feed(train_loader)):
            logits = model(x)
            loss = F.cross_entropy(logits, target)
            optimizer.zero_grad()
            loss.backward()
            if (i + 1) % 16 == 0:
                with mytorch.no_grad():
                    acc = accuracy_of(logits, target).mean().item()
                log(f"Epoch #{epoch}, step #{i}, accuracy: {acc * 100:0.2f}%, loss: {loss.item():0.4f}")
            optimizer.step()

        model.eval()
        correct = 0.0
        for x, target in feed(test_loader):
            with mytorch.no_grad():
                correct += accuracy_of(model(x), target).sum().item()
        accuracy = correct / test_size
        history.append(accuracy)
        log(f"Epoch #{epoch}, test accuracy: {accuracy * 100:0.2f}%")
        if save_ckpt:
            mytorch.save({"optimizer": optimizer.state_dict(), "model": model.state_dict(), "accuracy": accuracy, "epoch": epoch}, save_ckpt)
    return history


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--train-size", type=int, default=4096)
    ap.add_argument("--ckpt")
    ap.add_argument("--save-ckpt")
    a = ap.parse_args()
    train_mnist(a.device, a.epochs, a.train_size, ckpt=a.ckpt, save_ckpt=a.save_ckpt)
