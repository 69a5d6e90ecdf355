from mytorch_b200.tensor import Tensor


class Parameter(Tensor):
    """A tensor that requires a gradient; ``to`` returns a Parameter (mytorch/nn/parameter.py:4-10)."""

    def __init__(self, tensor: Tensor):
        super().__init__(tensor=tensor, requires_grad=True)

    def to(self, device):
        return Parameter(tensor=super().to(device))
