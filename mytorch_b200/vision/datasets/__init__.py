from .synthetic_mnist import SyntheticMNIST
