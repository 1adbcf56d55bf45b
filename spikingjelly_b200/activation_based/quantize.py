"""Quantisers with straight-through gradients.

Every rounding-type op is one table entry ``name -> forward``; the gradient passes through
unchanged.  ``clamp`` and ``multi_level_spike_count`` pass the gradient only inside a window.
Parity: ``spikingjelly/activation_based/quantize.py:4-883``.
"""
from __future__ import annotations

import torch

__all__ = ["round", "ceil", "floor", "clamp", "clamp_backward", "step_quantize", "step_quantize_forward",
           "multi_level_spike_count", "k_bit_quantize", "k_bit_quantize_forward", "affine_k_bit_quantize",
           "clamp_by_linear", "round_atgf", "ceil_atgf", "floor_atgf", "clamp_atgf", "step_quantize_atgf",
           "k_bit_quantize_atgf", "multi_level_spike_count_atgf"]


def _straight_through(name: str, fwd):
    """autograd.Function whose forward is ``fwd(x, *args)`` and whose backward is identity in ``x``."""

    def forward(ctx, x, *args):
        ctx.n_extra = len(args)
        return fwd(x, *args)

    def backward(ctx, grad_output):
        return (grad_output,) + (None,) * ctx.n_extra

    return type(name, (torch.autograd.Function,), {"forward": staticmethod(forward), "backward": staticmethod(backward)})


def step_quantize_forward(x: torch.Tensor, step: float):
    return torch.round(x / step) * step


def k_bit_quantize_forward(x: torch.Tensor, k: int):
    levels = float(1 << k) - 1.0
    return torch.round(x * levels) / levels


round_atgf = _straight_through("round_atgf", torch.round)
ceil_atgf = _straight_through("ceil_atgf", torch.ceil)
floor_atgf = _straight_through("floor_atgf", torch.floor)
step_quantize_atgf = _straight_through("step_quantize_atgf", step_quantize_forward)
k_bit_quantize_atgf = _straight_through("k_bit_quantize_atgf", k_bit_quantize_forward)


def round(x):  # noqa: A001 - mirrors the public name
    """``torch.round`` with identity gradient."""
    return round_atgf.apply(x)


def ceil(x):
    return ceil_atgf.apply(x)


def floor(x):
    return floor_atgf.apply(x)


def step_quantize(x, step: float):
    """Round to the nearest multiple of ``step`` (identity gradient)."""
    return step_quantize_atgf.apply(x, step)


def k_bit_quantize(x, k: int):
    """Quantise ``x in [0, 1]`` to ``2^k`` uniform levels (identity gradient)."""
    if k < 1:
        raise ValueError(f"k must be a positive integer, but got {k}")
    return k_bit_quantize_atgf.apply(x, k)


def affine_k_bit_quantize(x, k: int, w, b):
    return w * k_bit_quantize(x, k) + b


def clamp_backward(grad_output, x, min_value: float, max_value: float):
    return grad_output * ((x >= min_value) & (x <= max_value))


class clamp_atgf(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, min_value: float, max_value: float):
        ctx.save_for_backward(x)
        ctx.lo, ctx.hi = min_value, max_value
        return torch.clamp(x, min_value, max_value)

    @staticmethod
    def backward(ctx, grad_output):
        return clamp_backward(grad_output, ctx.saved_tensors[0], ctx.lo, ctx.hi), None, None


def clamp(x, min_value: float, max_value: float):
    """Clamp whose gradient is 1 inside ``[min, max]`` (borders included) and 0 outside."""
    return clamp_atgf.apply(x, min_value, max_value)


class multi_level_spike_count_atgf(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, max_spike_count: int, grad_min: float, grad_max: float):
        ctx.save_for_backward(x)
        ctx.lo, ctx.hi = grad_min, grad_max
        return torch.round(torch.clamp(x, 0, max_spike_count))

    @staticmethod
    def backward(ctx, grad_output):
        (x,) = ctx.saved_tensors
        mask = (x >= ctx.lo) & (x <= ctx.hi)
        return grad_output * mask.to(grad_output.dtype), None, None, None


def multi_level_spike_count(x, max_spike_count: int, grad_window=None):
    """Integer spike count ``round(clamp(x, 0, D))``; gradient 1 inside ``grad_window``."""
    max_spike_count = int(max_spike_count)
    lo, hi = (0.0, float(max_spike_count)) if grad_window is None else grad_window
    return multi_level_spike_count_atgf.apply(x, max_spike_count, lo, hi)


def clamp_by_linear(x, eps: float = 1e-5):
    """Affine map of ``x`` onto ``[0, 1)`` using its min and max."""
    x_min = torch.min(x)
    return (x - x_min) / (torch.max(x) + eps - x_min)
