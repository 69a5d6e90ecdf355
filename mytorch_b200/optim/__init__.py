from .optimizer import Optimizer
from .sgd import SGD
