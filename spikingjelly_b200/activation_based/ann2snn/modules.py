"""Calibration observers and voltage scalers of ANN-to-SNN conversion.

``VoltageHook`` watches the output of a ReLU during calibration and keeps a running estimate of its
scale (max, a percentile ``"99.9%"`` or a fraction of the max); after conversion the ReLU becomes
``VoltageScaler(1/s) -> IF neuron -> VoltageScaler(s)``.  ``ChannelVoltageScaler`` is the per-channel form.
Parity: ``spikingjelly/activation_based/ann2snn/modules.py:10-382``."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import base, functional

__all__ = ["VoltageHook", "VoltageScaler", "ChannelVoltageScaler"]

_BAD_MODE = "You have used a non-defined VoltageScale Method."


def _safe_quantile(x: torch.Tensor, quantile: float, dim: Optional[int] = None, max_elements: int = 1048576) -> torch.Tensor:
    """Linear-interpolated quantile through ``kthvalue`` (no size limit, unlike ``torch.quantile``);
    inputs longer than ``max_elements`` along the reduced axis are strided down first."""
    if not 0.0 <= quantile <= 1.0:
        raise ValueError("quantile must be in [0, 1].")
    if x.numel() == 0:
        raise ValueError("quantile input must not be empty.")
    if max_elements <= 0:
        raise ValueError("max_elements must be positive.")
    if dim is None:
        rows, shape = x.reshape(1, -1), ()
    else:
        dim = dim + x.dim() if dim < 0 else dim
        if not 0 <= dim < x.dim():
            raise ValueError("dim is out of range.")
        moved = x.movedim(dim, -1)
        rows, shape = moved.reshape(-1, moved.shape[-1]), moved.shape[:-1]
    if rows.shape[-1] > max_elements:
        rows = rows[:, ::math.ceil(rows.shape[-1] / max_elements)][:, :max_elements]
    rows = rows.contiguous()
    rank = quantile * (rows.shape[-1] - 1)
    lo, hi = int(math.floor(rank)), int(math.ceil(rank))
    low = rows.kthvalue(lo + 1, dim=1).values
    out = low if lo == hi else low + (rows.kthvalue(hi + 1, dim=1).values - low) * (rank - lo)
    return out.reshape(shape) if dim is not None else out.reshape(())


def _scale_statistic(x: torch.Tensor, mode, reduce_dim: Optional[int] = None) -> torch.Tensor:
    """max / percentile / fraction-of-max of ``x`` (over everything, or over ``reduce_dim`` of a 2-D view)."""
    def maximum(t):
        return t.max() if reduce_dim is None else t.max(dim=reduce_dim).values
    if isinstance(mode, str):
        if not mode:
            raise NotImplementedError(_BAD_MODE)
        if mode[-1] == "%":
            try:
                q = float(mode[:-1]) / 100.0
            except ValueError as exc:
                raise NotImplementedError(_BAD_MODE) from exc
            if not 0.0 <= q <= 1.0:
                raise NotImplementedError(_BAD_MODE)
            xf = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
            return _safe_quantile(xf, q, dim=reduce_dim).to(x.dtype)
        if mode.lower() == "max":
            return maximum(x)
        raise NotImplementedError(_BAD_MODE)
    if isinstance(mode, (int, float)) and not isinstance(mode, bool) and 0 < mode <= 1:
        return maximum(x) * mode
    raise NotImplementedError(_BAD_MODE)


class VoltageHook(nn.Module):
    """Identity that, in training mode, updates ``scale`` from its input (first batch: the statistic
    itself, then an exponential moving average with ``momentum``)."""

    def __init__(self, scale=1.0, momentum=0.1, mode="Max"):
        super().__init__()
        self.register_buffer("scale", torch.tensor(scale))
        self.mode, self.momentum, self.num_batches_tracked = mode, momentum, 0

    def forward(self, x):
        if not self.training:
            return x
        s_t = _scale_statistic(x.detach(), self.mode).detach()
        self.scale = s_t if self.num_batches_tracked == 0 else (1 - self.momentum) * self.scale + self.momentum * s_t
        self.num_batches_tracked += x.shape[0] if x.dim() > 0 else 1
        return x


class VoltageScaler(nn.Module, base.StepModule):
    def __init__(self, scale=1.0, step_mode: str = "s"):
        super().__init__()
        self.register_buffer("scale", torch.tensor(scale))
        self.step_mode = step_mode

    def _forward(self, x):
        return x * self.scale

    def forward(self, x):
        return self._forward(x) if self.step_mode == "s" else functional.seq_to_ann_forward(x, self._forward)

    def extra_repr(self):
        return f"{self.scale.item():f}, step_mode={self.step_mode}"


class ChannelVoltageScaler(nn.Module, base.StepModule):
    """Multiply by a positive scalar or a per-channel vector along ``channel_dim``."""

    def __init__(self, scale=1.0, channel_dim: int = 1, step_mode: str = "s"):
        super().__init__()
        if not isinstance(channel_dim, int):
            raise ValueError("channel_dim must be int.")
        s = torch.as_tensor(scale).detach().clone()
        if s.dim() > 1:
            raise ValueError("scale must be a scalar or a 1D tensor.")
        if s.numel() == 0:
            raise ValueError("scale must not be empty.")
        if not torch.isfinite(s).all() or (s <= 0).any():
            raise ValueError("scale must contain finite positive values.")
        self.register_buffer("scale", s)
        self.channel_dim, self.step_mode = channel_dim, step_mode

    def _forward(self, x: torch.Tensor) -> torch.Tensor:
        s = self.scale
        if s.dim() == 1:
            d = self.channel_dim + x.dim() if self.channel_dim < 0 else self.channel_dim
            if not 0 <= d < x.dim():
                raise ValueError("channel_dim is out of range for input.")
            if x.shape[d] != s.numel():
                raise ValueError(f"Input channel dimension does not match scale length: got {x.shape[d]} and {s.numel()}.")
            shape = [1] * x.dim()
            shape[d] = s.numel()
            s = s.reshape(shape)
        return x * s.to(dtype=x.dtype, device=x.device)

    def forward(self, x):
        return self._forward(x) if self.step_mode == "s" else functional.seq_to_ann_forward(x, self._forward)

    def extra_repr(self):
        return f"scale_shape={tuple(self.scale.shape)}, channel_dim={self.channel_dim}, step_mode={self.step_mode}"
