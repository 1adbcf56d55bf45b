"""Dropout for sequences: the mask is a memory, sampled at the first call after
``reset()`` and reused for every time step.

Parity: ``spikingjelly/activation_based/layer/dropout.py:15-415``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .. import base

__all__ = ["Dropout", "Dropout2d", "DropConnectLinear"]


class Dropout(base.MemoryModule):
    def __init__(self, p=0.5, step_mode="s"):
        super().__init__()
        self.step_mode = step_mode
        assert 0 <= p < 1
        self.register_memory("mask", None)
        self.p = p

    def extra_repr(self):
        return f"p={self.p}"

    def create_mask(self, x: Tensor) -> Tensor:
        return F.dropout(torch.ones_like(x), self.p, training=True)

    def _apply_mask(self, x, mask, like):
        if not self.training:
            return x, mask
        if mask is None:
            mask = self.create_mask(like)
        return x * mask, mask

    def single_step_functional_forward(self, inputs, states, **kwargs):
        y, mask = self._apply_mask(inputs[0], states[0], inputs[0])
        return (y,), (mask,)

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        y, mask = self._apply_mask(inputs[0], states[0], inputs[0][0])
        return (y,), (mask,)


class Dropout2d(Dropout):
    """Drops whole channels."""

    def __init__(self, p=0.2, step_mode="s"):
        super().__init__(p, step_mode)

    def create_mask(self, x: Tensor) -> Tensor:
        return F.dropout2d(torch.ones_like(x), self.p, training=True)


class DropConnectLinear(base.MemoryModule):
    """Linear layer with DropConnect: in training each sample gets its own Bernoulli mask on
    weights (and bias); in evaluation the output is the mean of ``samples_num`` draws from the
    Gaussian moment-matched pre-activation, pushed through ``activation``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, p: float = 0.5,
                 samples_num: int = 1024, invariant: bool = False, activation: Optional[nn.Module] = nn.ReLU(),
                 step_mode="s") -> None:
        super().__init__()
        self.step_mode = step_mode
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()
        self.p = p
        self.register_memory("dropped_w", None)
        if self.bias is not None:
            self.register_memory("dropped_b", None)
        self.samples_num, self.invariant, self.activation = samples_num, invariant, activation

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.weight.shape[1])
            nn.init.uniform_(self.bias, -bound, bound)

    def reset(self):
        super().reset()
        if hasattr(self.activation, "reset"):
            self.activation.reset()

    def drop(self, batch_size: int):
        keep_w = torch.rand(batch_size, *self.weight.shape, device=self.weight.device) >= self.p
        w = self.weight * keep_w
        if self.bias is None:
            return w, None
        keep_b = torch.rand(batch_size, *self.bias.shape, device=self.bias.device) >= self.p
        return w, self.bias * keep_b

    def single_step_functional_forward(self, inputs, states, **kwargs):
        x = inputs[0]
        w = states[0]
        b = states[1] if self.bias is not None else None
        if self.training:
            if not self.invariant or w is None:
                w, b = self.drop(x.shape[0])
            y = torch.bmm(w, x.unsqueeze(-1)).squeeze(-1)
            if self.bias is not None:
                y = y + b
            if self.activation is not None:
                y = self.activation(y)
            return (y,), ((w, b) if self.bias is not None else (w,))
        mu = (1 - self.p) * F.linear(x, self.weight, self.bias)
        var = self.p * (1 - self.p) * F.linear(x.square(), self.weight.square(),
                                               None if self.bias is None else self.bias.square())
        samples = torch.distributions.normal.Normal(mu, var.sqrt()).sample(torch.Size([self.samples_num]))
        if self.activation is not None:
            samples = self.activation(samples)
        return (samples.mean(dim=0),), states

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"p={self.p}, invariant={self.invariant}")
