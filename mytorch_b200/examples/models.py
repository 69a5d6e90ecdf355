"""Model definitions written against ``mytorch_b200.nn`` for the benchmark configurations.

The reference ships only a small MNIST CNN (``mytorch/examples/mnist.py:12-40``); the ResNets
below are built from the same six layer types.  Layers are created in a fixed order (stem,
then per block conv1, bn1, conv2, bn2, [downsample conv, bn], finally fc) because seeded
initialisation consumes one random draw per weight / bias tensor in creation order.
"""
import mytorch_b200.nn as nn
import mytorch_b200.nn.functional as F


class Flatten(nn.Module):
    def forward(self, x):
        return x.reshape((x.shape[0], -1))


def small_cnn(device="cpu"):
    """Conv(1,32,3)-ReLU-Conv(32,64,3)-ReLU-MaxPool(2)-flatten-Linear(9216,128)-ReLU-Linear(128,10)."""
    return nn.Sequential(
        nn.Conv2d(1, 32, 3, device=device), nn.ReLU(), nn.Conv2d(32, 64, 3, device=device), nn.ReLU(), nn.MaxPool2d(2, 2),
        Flatten(), nn.Linear(9216, 128, device=device), nn.ReLU(), nn.Linear(128, 10, device=device))


def _bn_relu(channels, fused, device):
    """(norm layer, relu-or-None): fused=True folds the ReLU into the BatchNorm kernel."""
    return (nn.BatchNormReLU2d(channels, device=device), None) if fused else (nn.BatchNorm2d(channels, device=device), nn.ReLU())


def _feed_batch_norm(*convs):
    """Mark convolutions whose output goes straight into a BatchNorm layer (see ``nn.Conv2d.feeds_batch_norm``)."""
    for conv in convs:
        conv.feeds_batch_norm = True


class BasicBlock(nn.Module):
    """fused=True uses the fused BatchNorm+ReLU and BatchNorm+add+ReLU operators (same arithmetic,
    fewer passes over memory); fused=False composes the six reference layer types one by one.
    conv_stats=True lets every convolution reduce the batch statistics its BatchNorm needs."""

    def __init__(self, cin, cout, stride, device="cpu", fused=True, conv_stats=True):
        super().__init__()
        self.fused = fused
        self.conv1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False, device=device)
        self.bn1 = nn.BatchNormReLU2d(cout, device=device) if fused else nn.BatchNorm2d(cout, device=device)
        self.conv2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False, device=device)
        self.bn2 = nn.BatchNormAddReLU2d(cout, device=device) if fused else nn.BatchNorm2d(cout, device=device)
        self.downsample = None
        if stride != 1 or cin != cout:
            self.downsample = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, 0, bias=False, device=device),
                                            nn.BatchNorm2d(cout, device=device))
        self.relu = nn.ReLU()
        if conv_stats:
            _feed_batch_norm(self.conv1, self.conv2, *([self.downsample._modules["0"]] if self.downsample is not None else []))

    def forward(self, x):
        # The projection shortcut is computed first: backward then meets it last, after conv1 has written a
        # gradient for every pixel of x, and the 1x1 / stride-2 convolution adds its own in place to the
        # pixels it reaches (instead of a zero-filled tensor that has to be added afterwards).
        shortcut = x if self.downsample is None else self.downsample(x)
        y = self.bn1(self.conv1(x))
        if not self.fused:
            y = self.relu(y)
        if self.fused:
            return self.bn2(self.conv2(y), shortcut)
        return self.relu(self.bn2(self.conv2(y)) + shortcut)


class ResNet18Cifar(nn.Module):
    """3x3 stride-1 stem without max-pool, stages of 2 BasicBlocks (strides 1/2/2/2), global
    average pool, Linear."""

    def __init__(self, widths=(64, 128, 256, 512), num_classes=10, device="cpu", fused=True, conv_stats=True):
        super().__init__()
        self.fused = fused
        self.conv1 = nn.Conv2d(3, widths[0], 3, 1, 1, bias=False, device=device)
        self.bn1 = nn.BatchNormReLU2d(widths[0], device=device) if fused else nn.BatchNorm2d(widths[0], device=device)
        self.relu = nn.ReLU()
        cin = widths[0]
        for si, wd in enumerate(widths):
            blocks = []
            for bi in range(2):
                blocks.append(BasicBlock(cin, wd, 2 if (si > 0 and bi == 0) else 1, device=device, fused=fused, conv_stats=conv_stats))
                cin = wd
            setattr(self, f"layer{si + 1}", nn.Sequential(*blocks))
        self.fc = nn.Linear(cin, num_classes, device=device)
        if conv_stats:
            _feed_batch_norm(self.conv1)

    def forward(self, x):
        x = self.bn1(self.conv1(x))
        if not self.fused:
            x = self.relu(x)
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(x.mean(dim=(2, 3)))


class Bottleneck(nn.Module):
    """1x1 reduce, 3x3 (carries the stride), 1x1 expand x4."""

    def __init__(self, cin, mid, stride, device="cpu"):
        super().__init__()
        cout = mid * 4
        self.conv1 = nn.Conv2d(cin, mid, 1, 1, 0, bias=False, device=device)
        self.bn1 = nn.BatchNorm2d(mid, device=device)
        self.conv2 = nn.Conv2d(mid, mid, 3, stride, 1, bias=False, device=device)
        self.bn2 = nn.BatchNorm2d(mid, device=device)
        self.conv3 = nn.Conv2d(mid, cout, 1, 1, 0, bias=False, device=device)
        self.bn3 = nn.BatchNorm2d(cout, device=device)
        self.downsample = None
        if stride != 1 or cin != cout:
            self.downsample = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, 0, bias=False, device=device),
                                            nn.BatchNorm2d(cout, device=device))
        self.relu = nn.ReLU()
        _feed_batch_norm(self.conv1, self.conv2, self.conv3, *([self.downsample._modules["0"]] if self.downsample is not None else []))

    def forward(self, x):
        y = self.relu(self.bn1(self.conv1(x)))
        y = self.relu(self.bn2(self.conv2(y)))
        y = self.bn3(self.conv3(y))
        shortcut = x if self.downsample is None else self.downsample(x)
        return self.relu(y + shortcut)


class ResNet50(nn.Module):
    """7x7/2 stem, 3x3/2 max-pool, bottleneck stages [3,4,6,3], global average pool, Linear."""

    def __init__(self, num_classes=1000, device="cpu"):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 64, 7, 2, 3, bias=False, device=device)
        _feed_batch_norm(self.conv1)
        self.bn1 = nn.BatchNorm2d(64, device=device)
        self.relu = nn.ReLU()
        self.maxpool = nn.MaxPool2d(3, 2, 1)
        cin = 64
        for si, (mid, count) in enumerate(zip((64, 128, 256, 512), (3, 4, 6, 3))):
            blocks = []
            for bi in range(count):
                blocks.append(Bottleneck(cin, mid, 2 if (si > 0 and bi == 0) else 1, device=device))
                cin = mid * 4
            setattr(self, f"layer{si + 1}", nn.Sequential(*blocks))
        self.fc = nn.Linear(cin, num_classes, device=device)

    def forward(self, x):
        x = self.maxpool(self.relu(self.bn1(self.conv1(x))))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(x.mean(dim=(2, 3)))


def bn_relu_pool(channels, device="cpu"):
    return nn.Sequential(nn.BatchNorm2d(channels, device=device), nn.ReLU(), nn.MaxPool2d(2, 2))
