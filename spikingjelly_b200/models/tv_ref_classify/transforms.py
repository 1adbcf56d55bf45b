"""Batch-level mixup and cutmix.  Inputs: float image batch ``[B, C, H, W]`` and int64 labels ``[B]``;
outputs: mixed images and soft labels ``[B, num_classes]``.  Pairs are formed by rolling the batch by
one, which needs no second permutation of the batch.

Parity: ``spikingjelly/activation_based/model/tv_ref_classify/transforms.py:10-312``.
"""
from __future__ import annotations

import math
from typing import Tuple

import torch
from torch import Tensor

__all__ = ["RandomMixup", "RandomCutmix"]


class _BatchMix(torch.nn.Module):
    def __init__(self, num_classes: int, p: float = 0.5, alpha: float = 1.0, inplace: bool = False):
        super().__init__()
        if num_classes < 1:
            raise ValueError(f"Please provide a valid positive value for the num_classes. Got num_classes={num_classes}")
        if alpha <= 0:
            raise ValueError("Alpha param can't be zero.")
        self.num_classes, self.p, self.alpha, self.inplace = num_classes, p, alpha, inplace

    def _check(self, batch: Tensor, target: Tensor) -> Tuple[Tensor, Tensor]:
        if batch.ndim != 4:
            raise ValueError(f"Batch ndim should be 4. Got {batch.ndim}")
        if target.ndim != 1:
            raise ValueError(f"Target ndim should be 1. Got {target.ndim}")
        if not batch.is_floating_point():
            raise TypeError(f"Batch dtype should be a float tensor. Got {batch.dtype}.")
        if target.dtype != torch.int64:
            raise TypeError(f"Target dtype should be torch.int64. Got {target.dtype}")
        if not self.inplace:
            batch, target = batch.clone(), target.clone()
        return batch, torch.nn.functional.one_hot(target, num_classes=self.num_classes).to(dtype=batch.dtype)

    def _lambda(self) -> float:
        return float(torch._sample_dirichlet(torch.tensor([self.alpha, self.alpha]))[0])

    def _mix(self, batch, target, batch_rolled, lam) -> Tensor:
        raise NotImplementedError

    def forward(self, batch: Tensor, target: Tensor) -> Tuple[Tensor, Tensor]:
        batch, target = self._check(batch, target)
        if torch.rand(1).item() >= self.p:
            return batch, target
        batch_rolled, target_rolled = batch.roll(1, 0), target.roll(1, 0)
        lam = self._mix(batch, batch_rolled, self._lambda())
        target_rolled.mul_(1.0 - lam)
        target.mul_(lam).add_(target_rolled)
        return batch, target

    def __repr__(self) -> str:
        return (f"{self.__class__.__name__}(num_classes={self.num_classes}, p={self.p}, alpha={self.alpha}, "
                f"inplace={self.inplace})")


class RandomMixup(_BatchMix):
    """mixup (Zhang et al., 2018): convex combination of image pairs with ``lambda ~ Beta(alpha, alpha)``."""

    def _mix(self, batch, batch_rolled, lam):
        batch_rolled.mul_(1.0 - lam)
        batch.mul_(lam).add_(batch_rolled)
        return lam


class RandomCutmix(_BatchMix):
    """CutMix (Yun et al., 2019): paste a random box of the partner image; the label weight is the
    area actually kept after clipping the box to the image."""

    def _mix(self, batch, batch_rolled, lam):
        h, w = batch.shape[-2:]
        cx, cy = int(torch.randint(w, (1,))), int(torch.randint(h, (1,)))
        half = 0.5 * math.sqrt(1.0 - lam)
        hw, hh = int(half * w), int(half * h)
        x1, y1 = max(cx - hw, 0), max(cy - hh, 0)
        x2, y2 = min(cx + hw, w), min(cy + hh, h)
        batch[:, :, y1:y2, x1:x2] = batch_rolled[:, :, y1:y2, x1:x2]
        return float(1.0 - (x2 - x1) * (y2 - y1) / (w * h))
