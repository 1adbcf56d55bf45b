"""Losses on per-step logits ``[T, N, C]`` for the CIFAR10-DVS example (``examples/memopt/loss.py`` of the reference)."""
import torch.nn as nn
import torch.nn.functional as F


class TMeanCrossEntropyLoss(nn.CrossEntropyLoss):
    """Cross entropy of the time-averaged logits."""

    def forward(self, y_seq, label):
        return super().forward(y_seq.mean(dim=0), label)


class TETLoss(nn.Module):
    """Temporal efficient training: the mean over steps of the per-step criterion, mixed with a pull of the logits
    towards ``mean``: ``(1 - lambda) * mean_t L(y[t], label) + lambda * MSE(y, mean)``."""

    def __init__(self, base_criterion=None, mean: float = 1.0, tet_lambda: float = 1e-3):
        super().__init__()
        self.base_criterion = nn.CrossEntropyLoss() if base_criterion is None else base_criterion
        self.mean, self.tet_lambda = mean, tet_lambda

    def base_criterion_loss(self, y, label):
        T = y.shape[0]
        if getattr(self.base_criterion, "reduction", None) == "mean":
            # equal step sizes: the mean over T of per-step means is the mean over the folded batch (one kernel, not T)
            return self.base_criterion(y.flatten(0, 1), label.repeat(T, *([1] * (label.dim() - 1))))
        return sum(self.base_criterion(y[t], label) for t in range(T)) / T

    def regularization_loss(self, y):
        return F.mse_loss(y, y.new_full((), self.mean).expand_as(y)) if self.tet_lambda != 0 else 0.0

    def forward(self, y, label):
        return (1.0 - self.tet_lambda) * self.base_criterion_loss(y, label) + self.tet_lambda * self.regularization_loss(y)
