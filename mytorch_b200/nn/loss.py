from mytorch_b200.nn.functional.cross_entropy import cross_entropy
from mytorch_b200.nn.module import Module


class CrossEntropyLoss(Module):
    """Mean softmax cross-entropy over a batch of logits [B, C] and int64 class indices [B]."""

    def forward(self, input, target):
        return cross_entropy(input, target)
