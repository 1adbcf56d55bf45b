"""Local threshold balancing: per-channel thresholds found online during calibration.  Each observed
batch raises a channel's threshold by twice the mean amount by which (non-negative) activations exceed
it, and the observer passes the activation *clipped* at the current threshold on to the next layer, so
that deeper layers are balanced against what the spiking layers before them can actually represent.
Every ReLU (with a directly following MaxPool2d moved before the neuron) becomes
``per-channel scale down -> half-threshold IF neuron -> per-channel scale up``.
Parity: ``spikingjelly/activation_based/ann2snn/recipes/local_threshold_balancing.py:28-325``."""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from .rate_coding import RateCodingRecipe

__all__ = ["LocalThresholdBalancingRecipe", "LocalThresholdBalancingHook"]


class LocalThresholdBalancingHook(nn.Module):
    def __init__(self, channel_dim: int = 1, eps: float = 1e-6) -> None:
        super().__init__()
        self.channel_dim, self.eps = channel_dim, float(eps)
        self.register_buffer("threshold", torch.empty(0))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() < 2:
            raise ValueError("LocalThresholdBalancingRecipe requires activation tensors with at least 2 dimensions.")
        d = self.channel_dim + x.dim() if self.channel_dim < 0 else self.channel_dim
        if not 0 <= d < x.dim():
            raise ValueError("channel_dim is out of range.")
        pos = torch.clamp(x, min=0)
        stat = pos.detach()
        stat = stat.float() if stat.dtype in (torch.float16, torch.bfloat16) else stat
        if self.threshold.numel() == 0:
            self.threshold = torch.zeros(x.shape[d], device=stat.device, dtype=stat.dtype)
        shape = [1] * x.dim()
        shape[d] = x.shape[d]
        th = self.threshold.to(stat)
        overflow = torch.clamp(stat - th.reshape(shape), min=0)
        th = torch.clamp(th + 2.0 * overflow.mean(dim=tuple(i for i in range(x.dim()) if i != d)), min=self.eps)
        self.threshold = th.detach()
        return torch.minimum(pos, th.to(x).reshape(shape))

    def compute_threshold(self) -> torch.Tensor:
        if self.threshold.numel() == 0:
            raise ValueError("No calibration activations have been recorded.")
        if not torch.isfinite(self.threshold).all() or (self.threshold <= 0).any():
            raise ValueError("Balanced thresholds must be finite positive values.")
        return self.threshold.detach()


class LocalThresholdBalancingRecipe(RateCodingRecipe):
    _channel_hook_type = LocalThresholdBalancingHook
    _channel_leaf = "ltb_hook_"

    def __init__(self, dataloader: Iterable, channel_dim: int = 1, fuse_flag: bool = True, eps: float = 1e-6) -> None:
        super().__init__(dataloader, mode="Max", fuse_flag=fuse_flag, channel_wise=True, channel_dim=channel_dim,
                         pre_spike_maxpool=True, half_threshold=True, eps=eps)

    def validate(self, converter) -> None:
        if self.dataloader is None:
            raise ValueError("LocalThresholdBalancingRecipe requires a dataloader.")
        if not isinstance(self.channel_dim, int):
            raise ValueError("channel_dim must be int.")
        if self.eps <= 0:
            raise ValueError("eps must be positive.")

    def _new_hook(self, index: int):
        return f"ltb_hook_{index}", LocalThresholdBalancingHook(self.channel_dim, self.eps)
