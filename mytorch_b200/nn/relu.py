from mytorch_b200.nn.functional.relu import relu
from mytorch_b200.nn.module import Module


class ReLU(Module):
    def forward(self, x):
        return relu(x)
