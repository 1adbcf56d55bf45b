"""Stateless steps of stateful layers (``functional/layer.py:13-200``)."""
from __future__ import annotations

from typing import Tuple, Union

import torch

__all__ = ["delay_step", "neunorm_step", "synapse_filter_step"]


def neunorm_step(in_spikes, state, weight, momentum: float, input_scale: float):
    """NeuNorm: ``x <- k x + scale * sum_c(spikes)``; output ``spikes - w * x``."""
    state = momentum * state + input_scale * in_spikes.sum(dim=1, keepdim=True)
    return in_spikes - weight * state, state


def delay_step(x, queue: Tuple[torch.Tensor, ...], delay_steps: int):
    """FIFO delay line: emits the input seen ``delay_steps`` calls ago (zeros before)."""
    if not isinstance(delay_steps, int) or delay_steps < 0:
        raise ValueError("delay_steps must be a non-negative integer")
    q = (*queue, x)
    if len(q) > delay_steps:
        return q[0], q[1:]
    return torch.zeros_like(x), q


def synapse_filter_step(x, out_i, reciprocal_tau: Union[float, torch.Tensor]):
    """First-order synaptic current: decays by ``1/tau`` without input, jumps by ``x``."""
    return out_i - (1.0 - x) * out_i * reciprocal_tau + x
