"""Miscellaneous layers (``spikingjelly/activation_based/layer/misc.py:22-629``)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ...logger import logger
from .. import base, functional

__all__ = ["SynapseFilter", "PrintShapeModule", "VotingLayer", "Delay", "SpikeCountToBinary", "TemporalBinSum"]


class SynapseFilter(base.MemoryModule):
    """Low-pass filter of a spike train: ``i <- i - (1 - s) i / tau + s``.  With
    ``learnable=True`` ``1/tau = sigmoid(w)`` and ``w`` is a parameter."""

    def __init__(self, tau=100.0, learnable=False, step_mode="s"):
        super().__init__()
        self.step_mode = step_mode
        self.learnable = learnable
        assert tau > 1
        if learnable:
            self.w = nn.Parameter(torch.as_tensor(-math.log(tau - 1)))
        else:
            self.tau = tau
        self.register_memory("out_i", 0.0)

    def extra_repr(self):
        tau = float(1.0 / self.w.detach().sigmoid()) if self.learnable else self.tau
        return f"tau={tau}, learnable={self.learnable}, step_mode={self.step_mode}"

    def materialize_states(self, inputs, states, step_mode):
        x = inputs[0]
        if step_mode == "m" and x.dim() > 0 and x.shape[0] > 0:
            x = x[0]
        s = states[0]
        if isinstance(s, float):
            s = torch.full_like(x, s)
        elif isinstance(s, Tensor):
            if s.shape != x.shape:
                s = torch.zeros_like(x)
            elif s.dtype != x.dtype or s.device != x.device:
                s = s.to(dtype=x.dtype, device=x.device)
        return (s,)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        inv_tau = self.w.sigmoid() if self.learnable else 1.0 / self.tau
        out = functional.synapse_filter_step(inputs[0], states[0], inv_tau)
        return (out,), (out,)


class PrintShapeModule(nn.Module):
    """Identity that logs the shape of what passes through (debug level)."""

    def __init__(self, ext_str="PrintShapeModule"):
        super().__init__()
        self.ext_str = ext_str

    def forward(self, x: Tensor):
        logger.debug("%s shape=%s", self.ext_str, x.shape)
        return x


class VotingLayer(nn.Module, base.StepModule):
    """Average groups of ``voting_size`` consecutive output neurons into one class score."""

    def __init__(self, voting_size: int = 10, step_mode="s"):
        super().__init__()
        self.voting_size = voting_size
        self.step_mode = step_mode

    def extra_repr(self):
        return f"voting_size={self.voting_size}, step_mode={self.step_mode}"

    def single_step_forward(self, x: torch.Tensor):
        return F.avg_pool1d(x.unsqueeze(1), self.voting_size, self.voting_size).squeeze(1)

    def forward(self, x: torch.Tensor):
        if self.step_mode == "s":
            return self.single_step_forward(x)
        return functional.seq_to_ann_forward(x, self.single_step_forward)


class Delay(base.MemoryModule):
    """Delay line of ``delay_steps`` steps (memory ``queue``)."""

    def __init__(self, delay_steps: int, step_mode="s"):
        super().__init__()
        assert isinstance(delay_steps, int) and delay_steps >= 0
        self._delay_steps = delay_steps
        self.step_mode = step_mode
        self.register_memory("queue", [])

    @property
    def delay_steps(self):
        return self._delay_steps

    def single_step_functional_forward(self, inputs, states, **kwargs):
        y, q = functional.delay_step(inputs[0], tuple(states[0]), self.delay_steps)
        return (y,), (list(q),)

    def single_step_forward(self, x: Tensor) -> Tensor:
        (y,), (q,) = self.single_step_functional_forward((x,), (self.queue,))
        self.queue[:] = q
        return y

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        q, ys = tuple(states[0]), []
        for x in inputs[0]:
            y, q = functional.delay_step(x, q, self.delay_steps)
            ys.append(y)
        return (torch.stack(ys),), (list(q),)


def _check_slots(num_slots):
    if num_slots < 1:
        raise ValueError("num_slots must be >= 1.")


class SpikeCountToBinary(nn.Module, base.MultiStepModule):
    """Expand integer spike counts ``[T, N, *]`` into ``num_slots`` binary sub-steps
    ``[T*num_slots, N, *]`` (count ``c`` becomes ``c`` ones followed by zeros).  Identity in
    training unless ``always_convert``; the gradient flows as ``count / num_slots``."""

    def __init__(self, num_slots: int, always_convert: bool = False) -> None:
        super().__init__()
        _check_slots(num_slots)
        self.num_slots, self.always_convert = num_slots, always_convert
        self._step_mode = "m"

    def forward(self, x_seq: torch.Tensor) -> torch.Tensor:
        if not self.always_convert and self.training:
            return x_seq
        if x_seq.ndim < 2 or x_seq.shape[0] == 0:
            raise ValueError("x_seq must have shape [T, N, *] with T > 0.")
        counts = x_seq.unsqueeze(1)
        slots = torch.arange(self.num_slots, device=x_seq.device).view(1, -1, *((1,) * (x_seq.ndim - 1)))
        hard = (slots < counts).to(x_seq.dtype)
        proxy = counts / self.num_slots
        return (hard + (proxy - proxy.detach())).flatten(0, 1)


class TemporalBinSum(nn.Module, base.MultiStepModule):
    """Inverse of :class:`SpikeCountToBinary`: sum every ``num_slots`` steps (zero padded)."""

    def __init__(self, num_slots: int, always_convert: bool = False) -> None:
        super().__init__()
        _check_slots(num_slots)
        self.num_slots, self.always_convert = num_slots, always_convert
        self._step_mode = "m"

    def forward(self, x_seq: torch.Tensor) -> torch.Tensor:
        if not self.always_convert and self.training:
            return x_seq
        if x_seq.ndim < 2 or x_seq.shape[0] == 0:
            raise ValueError("x_seq must have shape [T, N, *] with T > 0.")
        rem = x_seq.shape[0] % self.num_slots
        if rem:
            x_seq = torch.cat((x_seq, x_seq.new_zeros((self.num_slots - rem, *x_seq.shape[1:]))))
        return x_seq.reshape(-1, self.num_slots, *x_seq.shape[1:]).sum(dim=1)
