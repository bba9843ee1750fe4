"""The MLP classifier of the first benchmark configuration: 784 -> 128 ReLU -> 10 with
softmax cross-entropy and SGD. The reference's ``models/mlp.cpp`` is empty, so the model is
composed from the same parts a user of the reference would use: ``Linear`` (src/linear.h),
``relu`` (src/activations.h), ``softmax`` + ``cross_entropy`` (src/softmax.h, src/loss.h) and
``SGD`` (src/optimizers.h)."""
from __future__ import annotations

from ..ops import functional as F
from ..tensor import Tensor
from .layers import Linear, Module


class MLP(Module):
    def __init__(self, d_in: int = 784, d_hidden: int = 128, n_classes: int = 10, dtype=None, device=None,
                 fused: bool = True):
        self.fc1 = Linear(d_in, d_hidden, dtype=dtype, device=device, fused=fused)
        self.fc2 = Linear(d_hidden, n_classes, dtype=dtype, device=device, fused=fused)
        self.n_classes = n_classes
        self.fused = fused

    def forward(self, x: Tensor) -> Tensor:
        return self.fc2.forward(self.fc1.forward(x, act="relu"))

    def loss(self, x: Tensor, labels, reduction: str = "reference") -> Tensor:
        """Cross-entropy of softmax(logits) against integer labels. ``reduction="reference"``
        divides by rows * classes as the reference's loss does (src/loss.h:32,43)."""
        logits = self.forward(x)
        if self.fused:
            return F.softmax_cross_entropy(logits, labels, reduction=reduction)
        probs = F.softmax(logits)
        loss = F.cross_entropy(probs, F.one_hot(labels, self.n_classes))
        return loss if reduction == "reference" else F.mul_scalar(loss, float(self.n_classes))

    def parameters(self) -> list[Tensor]:
        return self.fc1.parameters() + self.fc2.parameters()
