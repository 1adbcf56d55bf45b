"""Parallel spiking neurons: the membrane potential of all time steps is one matrix product
``H = W [T, T] @ X [T, N] + b``, so there is no sequential dependence over time.

Parity: ``neuron/psn.py`` — ``PSN`` :13-99, ``MaskedPSN`` :102-306, ``SlidingPSN`` :309-474.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import base, functional, surrogate

__all__ = ["PSN", "MaskedPSN", "SlidingPSN"]


def _psn_params(T: int):
    weight = nn.Parameter(torch.zeros([T, T]))
    bias = nn.Parameter(torch.zeros([T, 1]))
    nn.init.kaiming_uniform_(weight, a=math.sqrt(5))
    nn.init.constant_(bias, -1.0)
    return weight, bias


def _fused_spikes(x_seq, weight, bias, sg):
    """The one-kernel path (``ops/psn.py``) when the input qualifies, else None."""
    if not (torch.is_tensor(x_seq) and x_seq.is_cuda):
        return None
    from ...ops import psn as psn_op
    spec = surrogate.surrogate_spec(sg)
    if not psn_op.supported(x_seq, spec) or x_seq.shape[0] != weight.shape[0]:
        return None
    if torch.is_autocast_enabled("cuda") and x_seq.dtype == torch.float32:
        x_seq = x_seq.to(torch.get_autocast_dtype("cuda"))
    return psn_op.psn_spikes(x_seq, weight, bias, spec, sg)


class PSN(nn.Module, base.MultiStepModule):
    def __init__(self, T: int, surrogate_function=surrogate.ATan()):
        super().__init__()
        self._step_mode = "m"
        self.T = T
        self.surrogate_function = surrogate_function
        self.weight, self.bias = _psn_params(T)

    def forward(self, x_seq: torch.Tensor):
        fused = _fused_spikes(x_seq, self.weight, self.bias, self.surrogate_function)
        if fused is not None:
            return fused
        h = torch.addmm(self.bias, self.weight, x_seq.flatten(1))
        return self.surrogate_function(h).view(x_seq.shape)

    def extra_repr(self):
        return super().extra_repr() + f"T={self.T}, "


class MaskedPSN(base.MemoryModule):
    """PSN whose weight is masked to the last ``k`` steps; ``lambda_`` in [0, 1] blends from
    the full matrix (0) to the banded one (1) during training."""

    def __init__(self, k: int, T: int, lambda_init: float = 0.0, surrogate_function=surrogate.ATan(),
                 step_mode: str = "s"):
        super().__init__()
        self.register_memory("time_step", 0)
        self.register_memory("queue", [])
        self.step_mode = step_mode
        self.k, self.T = k, T
        self.surrogate_function = surrogate_function
        self.register_buffer("_lambda_", torch.as_tensor(lambda_init))
        self.weight, self.bias = _psn_params(T)
        ones = torch.ones([T, T])
        self.register_buffer("mask0", torch.tril(ones) * torch.triu(ones, -(k - 1)))
        self.register_buffer("mask1", ones)

    @staticmethod
    def gen_masked_weight(lambda_, mask0, mask1, weight):
        return (lambda_ * mask0 + (1.0 - lambda_) * mask1) * weight

    def masked_weight(self):
        if self.lambda_ >= 1.0:
            return self.weight * self.mask0
        return self.gen_masked_weight(self.lambda_, self.mask0, self.mask1, self.weight)

    @property
    def lambda_(self):
        return self._lambda_

    @lambda_.setter
    def lambda_(self, value: float):
        torch.fill_(self.lambda_, value)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        t = states[0]
        if self.lambda_ < 1.0:
            raise ValueError("The masked PSN can not work in single-step mode when k < 1!")
        if t + 1 > self.T:
            raise OverflowError(f"The MaskedPSN(T={self.T}) has run {t + 1} time-steps!")
        spike, t, q = functional.masked_psn_step(inputs[0], t, tuple(states[1]), self.masked_weight(), self.bias,
                                                 self.k, self.surrogate_function)
        return (spike,), (t, list(q))

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        x_seq = inputs[0]
        assert x_seq.shape[0] == self.T
        fused = _fused_spikes(x_seq, self.masked_weight(), self.bias, self.surrogate_function)
        if fused is not None:
            return (fused,), states
        h = torch.addmm(self.bias, self.masked_weight(), x_seq.flatten(1))
        return (self.surrogate_function(h).view(x_seq.shape),), states

    def extra_repr(self):
        return super().extra_repr() + f", lambda_={self.lambda_}, T={self.T}"


class SlidingPSN(base.MemoryModule):
    """PSN with one shared weight vector of order ``k`` slid over time (any ``T``).
    ``backend``: ``"gemm"`` (banded Toeplitz matrix) or ``"conv"`` (causal 1-D convolution)."""

    def __init__(self, k: int, exp_init: bool = True, surrogate_function=surrogate.ATan(), step_mode: str = "s",
                 backend: str = "gemm"):
        super().__init__()
        self.register_memory("queue", [])
        self.step_mode = step_mode
        self.k = k
        self.surrogate_function = surrogate_function
        self.backend = backend
        if exp_init:
            weight = torch.tensor([2.0 ** (i - (k - 1)) for i in range(k)])
        else:
            weight = torch.ones([1, k])
            nn.init.kaiming_uniform_(weight, a=math.sqrt(5))
            weight = weight[0]
        self.weight = nn.Parameter(weight)
        self.bias = nn.Parameter(torch.as_tensor(-1.0))

    @property
    def supported_backends(self):
        return "gemm", "conv"

    def gen_gemm_weight(self, T: int):
        """Lower-banded Toeplitz ``[T, T]``: row ``i`` holds the last ``min(i+1, k)`` taps."""
        idx = torch.arange(T, device=self.weight.device)
        lag = idx.view(-1, 1) - idx.view(1, -1)                   # i - j
        valid = (lag >= 0) & (lag < self.k)
        taps = self.weight[(self.k - 1 - lag).clamp(0, self.k - 1)]
        return torch.where(valid, taps, torch.zeros((), device=taps.device, dtype=taps.dtype))

    def single_step_functional_forward(self, inputs, states, **kwargs):
        spike, q = functional.sliding_psn_step(inputs[0], tuple(states[0]), self.weight, self.bias,
                                               self.surrogate_function)
        return (spike,), (list(q),)

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        x_seq = inputs[0]
        if self.backend == "gemm":
            w = self.gen_gemm_weight(x_seq.shape[0])
            fused = _fused_spikes(x_seq, w, self.bias.reshape(-1).expand(x_seq.shape[0]), self.surrogate_function)
            if fused is not None:
                return (fused,), states
            h = torch.addmm(self.bias, w, x_seq.flatten(1)).view(x_seq.shape)
            return (self.surrogate_function(h),), states
        if self.backend == "conv":
            shape = x_seq.shape
            seq = F.pad(x_seq.flatten(1).t().unsqueeze(1), pad=(self.k - 1, 0))
            seq = F.conv1d(seq, self.weight.view(1, 1, -1), stride=1).squeeze(1).t().view(shape)
            return (self.surrogate_function(seq + self.bias),), states
        raise NotImplementedError(self.backend)

    def extra_repr(self):
        return super().extra_repr() + f", order={self.k}"
