from mytorch_b200.ops.elementwise_ops import _relu


def relu(x):
    return _relu(x)
