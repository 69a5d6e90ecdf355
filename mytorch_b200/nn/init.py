"""Kaiming-uniform initialisation (``mytorch/nn/init.py:1-17``)."""


def _calculate_fan_in_and_fan_out(tensor):
    receptive = 1
    for d in tensor.shape[2:]:
        receptive *= d
    return tensor.shape[1] * receptive, tensor.shape[0] * receptive


def kaiming_uniform_(tensor, a=0, mode="fan_in"):
    fan_in, fan_out = _calculate_fan_in_and_fan_out(tensor)
    fan = fan_in if mode == "fan_in" else fan_out
    bound = (6 / (1 + a ** 2) / fan) ** 0.5
    tensor.uniform_(-bound, bound)
