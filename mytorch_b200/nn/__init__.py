from .batch_norm import BatchNorm1d, BatchNorm2d, BatchNormAddReLU2d, BatchNormReLU2d
from .conv import Conv2d
from .linear import Linear
from .max_pool import MaxPool2d
from .module import Module
from .parameter import Parameter
from .relu import ReLU
from .sequential import Sequential
from .loss import CrossEntropyLoss
