"""Spike encoders: turn real-valued inputs into spike trains.

Parity: ``spikingjelly/activation_based/encoding.py:22-951``.
"""
from __future__ import annotations

import math
from abc import abstractmethod

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import base, functional, neuron, surrogate

__all__ = ["StatelessEncoder", "StatefulEncoder", "PeriodicEncoder", "LatencyEncoder", "PoissonEncoder",
           "WeightedPhaseEncoder", "PopSpikeEncoderDeterministic", "PopSpikeEncoderRandom", "PopEncoder"]


class StatelessEncoder(nn.Module, base.StepModule):
    """Encoder whose output at a step depends only on that step's input."""

    def __init__(self, step_mode="s"):
        super().__init__()
        self.step_mode = step_mode

    @abstractmethod
    def forward(self, x: torch.Tensor):
        raise NotImplementedError


class StatefulEncoder(base.MemoryModule):
    """Encoder that computes a length-``T`` spike train at the first call (memory ``spike``)
    and then plays it back one step per call, cyclically (memory ``t``)."""

    def __init__(self, T: int, step_mode="s"):
        super().__init__()
        self.step_mode = step_mode
        assert isinstance(T, int) and T >= 1
        self.T = T
        self.register_memory("spike", None)
        self.register_memory("t", 0)

    def single_step_forward(self, x: torch.Tensor = None):
        return super().single_step_forward(x)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        spike, t = states
        if spike is None:
            spike = self.single_step_encode(inputs[0])
        return (spike[t],), (spike, (t + 1) % spike.shape[0])

    @abstractmethod
    def single_step_encode(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def extra_repr(self) -> str:
        return f"T={self.T}"


class PeriodicEncoder(StatefulEncoder):
    """Replays a given spike tensor ``[T, *]`` periodically."""

    def __init__(self, spike: torch.Tensor, step_mode="s"):
        super().__init__(spike.shape[0], step_mode)

    def single_step_encode(self, spike):
        return spike


class LatencyEncoder(StatefulEncoder):
    """Stronger input -> earlier single spike.  ``linear``: ``t = (T-1)(1-x)``;
    ``log``: ``t = T-1 - ln(alpha x + 1)`` with ``alpha = e^{T-1} - 1``."""

    def __init__(self, T: int, enc_function="linear", step_mode="s"):
        super().__init__(T, step_mode)
        if enc_function == "log":
            self.alpha = math.exp(T - 1.0) - 1.0
        elif enc_function != "linear":
            raise NotImplementedError
        self.enc_function = enc_function

    def single_step_encode(self, x):
        if self.enc_function == "log":
            t_f = (self.T - 1.0 - torch.log(self.alpha * x + 1.0)).round().long()
        else:
            t_f = ((self.T - 1.0) * (1.0 - x)).round().long()
        return F.one_hot(t_f, num_classes=self.T).to(x).movedim(-1, 0)


class PoissonEncoder(StatelessEncoder):
    """Bernoulli spikes with firing probability ``x`` (``x`` in ``[0, 1]``)."""

    def forward(self, x: torch.Tensor):
        return torch.rand_like(x).le(x).to(x)


class WeightedPhaseEncoder(StatefulEncoder):
    """Binary expansion: phase ``i`` carries weight ``2^-(i+1)``."""

    def __init__(self, K: int, step_mode="s"):
        super().__init__(K, step_mode)

    def single_step_encode(self, x):
        assert (x >= 0).all() and (x <= 1 - 2 ** (-self.T)).all()
        rest = x.clone()
        spike = torch.empty((self.T,) + x.shape, device=x.device)
        w = 0.5
        for i in range(self.T):
            spike[i] = rest >= w
            rest -= w * spike[i]
            w *= 0.5
        return spike


class _PopBase(nn.Module):
    """Gaussian receptive-field population code: ``pop_dim`` neurons per observation dim."""

    def __init__(self, obs_dim, pop_dim, spike_ts, mean_range, std):
        super().__init__()
        self.obs_dim, self.pop_dim, self.spike_ts = obs_dim, pop_dim, spike_ts
        self.encoder_neuron_num = obs_dim * pop_dim
        mean = torch.linspace(mean_range[0], mean_range[1], pop_dim).expand(1, obs_dim, pop_dim).clone()
        self.mean = nn.Parameter(mean)
        self.std = nn.Parameter(torch.full_like(mean, std))

    def activity(self, obs):
        obs = obs.view(-1, self.obs_dim, 1)
        return torch.exp(-0.5 * ((obs - self.mean) / self.std).square()).flatten(1)


class PopSpikeEncoderDeterministic(_PopBase):
    """Population activity drives soft-reset IF neurons for ``spike_ts`` steps."""

    def __init__(self, obs_dim, pop_dim, spike_ts, mean_range, std):
        super().__init__(obs_dim, pop_dim, spike_ts, mean_range, std)
        self.neurons = neuron.IFNode(v_threshold=0.999, v_reset=None,
                                     surrogate_function=surrogate.DeterministicPass(), detach_reset=True)
        functional.set_step_mode(self, step_mode="m")
        functional.set_backend(self, backend="torch")

    def forward(self, obs):
        act = self.activity(obs)
        return self.neurons(act.unsqueeze(0).repeat(self.spike_ts, 1, 1))


class PopSpikeEncoderRandom(_PopBase):
    """Population activity is the Bernoulli rate of each step's spikes."""

    def __init__(self, obs_dim, pop_dim, spike_ts, mean_range, std):
        super().__init__(obs_dim, pop_dim, spike_ts, mean_range, std)
        self.pseudo_spike = surrogate.poisson_pass.apply

    def forward(self, obs):
        act = self.activity(obs)
        return self.pseudo_spike(act.unsqueeze(0).expand(self.spike_ts, *act.shape))


class PopEncoder(_PopBase):
    """Analog population activity repeated over ``spike_ts`` steps."""

    def forward(self, obs):
        return self.activity(obs).unsqueeze(0).repeat(self.spike_ts, 1, 1)
