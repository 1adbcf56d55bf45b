"""Population-decoder neurons for spiking reinforcement learning: inter-layer-connection (ILC)
neurons whose spikes feed back laterally within each action's population, and noisy variants
with colored-noise exploration.

Parity: ``neuron/inter_layer_connection.py:13-629``, ``neuron/noisy.py:26-542``.
"""
from __future__ import annotations

import math
from abc import abstractmethod
from typing import Iterable, Optional, Union

import numpy as np
import torch
import torch.nn as nn

from .. import base, surrogate

__all__ = ["ILCBaseNode", "ILCIFNode", "ILCLIFNode", "ILCCUBALIFNode", "powerlaw_psd_gaussian", "NoisyBaseNode",
           "NoisyCUBALIFNode", "NoisyILCBaseNode", "NoisyILCCUBALIFNode", "NoisyNonSpikingBaseNode",
           "NoisyNonSpikingIFNode"]


class _Dynamics:
    """charge / fire / reset on attributes ``v`` (and ``c`` for current-based neurons)."""

    def neuronal_fire(self):
        return self.surrogate_function(self.v - self.v_threshold)

    def neuronal_reset(self, spike):
        if self.v_reset is None:
            self.v = self.v - spike * self.v_threshold
        else:
            self.v = (1.0 - spike) * self.v + spike * self.v_reset

    def init_tensor(self, data: torch.Tensor):
        self.v = torch.full_like(data, fill_value=self.v_reset)


class _CubaCharge:
    def neuronal_charge(self, x):
        self.c = self.c * self.c_decay + x
        self.v = self.v * self.v_decay + self.c

    def init_tensor(self, data):
        self.c = torch.zeros_like(data)
        self.v = torch.full_like(data, fill_value=self.v_reset)


# The sequence-only nodes of this file set no ``_step_mode``: as in the reference, ``hasattr(node, "step_mode")`` is False and
# ``functional.set_step_mode`` passes them by.
class ILCBaseNode(_Dynamics, nn.Module, base.MultiStepModule):
    """Each action owns ``dec_pop_dim`` neurons; the spikes of step ``t`` are mixed within each
    population by a grouped ``Conv1d`` (``conn``) and added to the input of step ``t + 1``."""

    def __init__(self, act_dim, dec_pop_dim, v_threshold: float = 1.0, v_reset: Optional[float] = 0.0,
                 surrogate_function=surrogate.Rect()):
        assert isinstance(v_reset, float) or v_reset is None
        assert isinstance(v_threshold, float)
        super().__init__()
        self.act_dim, self.dec_pop_dim, self.out_pop_dim = act_dim, dec_pop_dim, act_dim * dec_pop_dim
        self.conn = nn.Conv1d(act_dim, self.out_pop_dim, dec_pop_dim, groups=act_dim)
        self.v_threshold, self.v_reset, self.surrogate_function = v_threshold, v_reset, surrogate_function

    @abstractmethod
    def neuronal_charge(self, x):
        raise NotImplementedError

    def forward(self, x_seq: torch.Tensor):
        self.init_tensor(x_seq[0].detach())
        T = x_seq.shape[0]
        out, lateral = [], None
        for t in range(T):
            x = x_seq[t] if lateral is None else x_seq[t] + lateral
            self.neuronal_charge(x)
            spike = self.neuronal_fire()
            self.neuronal_reset(spike)
            out.append(spike)
            lateral = None
            if t < T - 1:
                lateral = self.conn(spike.view(-1, self.act_dim, self.dec_pop_dim)).view(-1, self.out_pop_dim)
        return torch.stack(out)


class ILCIFNode(ILCBaseNode):
    def neuronal_charge(self, x):
        self.v = self.v + x


class ILCLIFNode(ILCBaseNode):
    def __init__(self, act_dim, dec_pop_dim, v_decay: float = 0.75, v_threshold: float = 1.0,
                 v_reset: Optional[float] = 0.0, surrogate_function=surrogate.Rect()):
        super().__init__(act_dim, dec_pop_dim, v_threshold, v_reset, surrogate_function)
        self.v_decay = v_decay

    def neuronal_charge(self, x):
        self.v = self.v * self.v_decay + x


class ILCCUBALIFNode(_CubaCharge, ILCBaseNode):
    def __init__(self, act_dim, dec_pop_dim, c_decay: float = 0.5, v_decay: float = 0.75, v_threshold: float = 0.5,
                 v_reset: Optional[float] = 0.0, surrogate_function=surrogate.Rect()):
        super().__init__(act_dim, dec_pop_dim, v_threshold, v_reset, surrogate_function)
        self.c_decay, self.v_decay = c_decay, v_decay


def powerlaw_psd_gaussian(exponent: float, size: Union[int, Iterable[int]], fmin: float = 0.0, random_state=None):
    """Gaussian noise with power spectral density ``1 / f^exponent`` along the last axis, unit
    variance (Timmer & Koenig 1995): white spectrum shaped in the frequency domain, then an
    inverse real FFT.  ``fmin`` in ``[0, 0.5]`` is the low-frequency cut-off."""
    size = [int(size)] if isinstance(size, (int, np.integer)) else list(size)
    n = size[-1]
    if not 0 <= fmin <= 0.5:
        raise ValueError("fmin must be chosen between 0 and 0.5.")
    fmin = max(fmin, 1.0 / n)
    freqs = np.fft.rfftfreq(n)
    scale = freqs.copy()
    cut = int(np.sum(scale < fmin))
    if cut and cut < len(scale):
        scale[:cut] = scale[cut]
    scale = scale ** (-exponent / 2.0)
    w = scale[1:].copy()
    w[-1] *= (1 + (n % 2)) / 2.0
    sigma = 2 * np.sqrt(np.sum(w ** 2)) / n
    size[-1] = len(freqs)
    scale = scale[(np.newaxis,) * (len(size) - 1) + (Ellipsis,)]
    if random_state is None or isinstance(random_state, (int, np.integer)):
        normal = np.random.default_rng(random_state).normal
    elif isinstance(random_state, (np.random.Generator, np.random.RandomState)):
        normal = random_state.normal
    else:
        raise ValueError("random_state must be one of integer, numpy.random.Generator, numpy.random.Randomstate")
    re, im = normal(scale=scale, size=size), normal(scale=scale, size=size)
    if n % 2 == 0:
        im[..., -1] = 0
        re[..., -1] *= np.sqrt(2)
    im[..., 0] = 0
    re[..., 0] *= np.sqrt(2)
    return np.fft.irfft(re + 1j * im, n=n, axis=-1) / sigma


def _noise_table(beta, num_node, num_rl_step, T):
    eps = powerlaw_psd_gaussian(beta, [num_node, num_rl_step * T]).reshape(num_node, num_rl_step, T)
    return torch.as_tensor(eps, dtype=torch.float).permute(1, 2, 0)      # [rl step, T, node]


class NoisyBaseNode(_Dynamics, nn.Module, base.MultiStepModule):
    """Spiking population with colored noise injected into the input current (``sigma_v``) and
    added to the output spikes (``sigma_s``).  ``reset_noise`` pre-samples a noise table for an
    episode; ``load_colored_noise`` replays stored noise when evaluating a sampled batch."""

    def __init__(self, num_node, is_training: bool = True, T: int = 5, sigma_init: float = 0.5, beta: float = 0.0,
                 v_threshold: float = 0.5, v_reset: Optional[float] = 0.0, surrogate_function=surrogate.Rect()):
        assert isinstance(v_reset, float) or v_reset is None
        assert isinstance(v_threshold, float)
        super().__init__()
        self.num_node, self.is_training, self.T, self.beta = num_node, is_training, T, beta
        self.sigma_v = self.sigma_s = sigma_init / math.sqrt(num_node)
        self.cn_v = self.cn_s = None
        self.v_threshold, self.v_reset, self.surrogate_function = v_threshold, v_reset, surrogate_function

    @abstractmethod
    def neuronal_charge(self, x):
        raise NotImplementedError

    def _after_spike(self, t: int, spike):
        return None

    def forward(self, x_seq: torch.Tensor):
        self.init_tensor(x_seq[0])
        if self.is_training and (self.cn_v is None or self.cn_s is None):
            self.noise_step += 1
        out, recurrent = [], None
        for t in range(self.T):
            x = x_seq[t] if recurrent is None else x_seq[t] + recurrent
            if self.is_training:
                nv = self.eps_v_seq[self.noise_step][t].to(x_seq.device) if self.cn_v is None else self.cn_v[:, t]
                x = x + self.sigma_v * nv
            self.neuronal_charge(x)
            spike = self.neuronal_fire()
            self.neuronal_reset(spike)
            if self.is_training:
                ns = self.eps_s_seq[self.noise_step][t].to(x_seq.device) if self.cn_s is None else self.cn_s[:, t]
                spike = spike + self.sigma_s * ns
            out.append(spike)
            recurrent = self._after_spike(t, spike)
        return torch.stack(out)

    def reset_noise(self, num_rl_step):
        self.eps_v_seq = _noise_table(self.beta, self.num_node, num_rl_step, self.T)
        self.eps_s_seq = _noise_table(self.beta, self.num_node, num_rl_step, self.T)
        self.noise_step = -1

    def get_colored_noise(self):
        return torch.cat([self.eps_v_seq[self.noise_step], self.eps_s_seq[self.noise_step]], dim=1)

    def load_colored_noise(self, cn):
        self.cn_v, self.cn_s = cn[:, :, : self.num_node], cn[:, :, self.num_node:]

    def cancel_load(self):
        self.cn_v = self.cn_s = None


class NoisyCUBALIFNode(_CubaCharge, NoisyBaseNode):
    def __init__(self, num_node, c_decay: float = 0.5, v_decay: float = 0.75, is_training: bool = True, T: int = 5,
                 sigma_init: float = 0.5, beta: float = 0.0, v_threshold: float = 0.5, v_reset: Optional[float] = 0.0,
                 surrogate_function=surrogate.Rect()):
        super().__init__(num_node, is_training, T, sigma_init, beta, v_threshold, v_reset, surrogate_function)
        self.c_decay, self.v_decay = c_decay, v_decay


class NoisyILCBaseNode(NoisyBaseNode):
    def __init__(self, act_dim, dec_pop_dim, is_training: bool = True, T: int = 5, sigma_init: float = 0.5,
                 beta: float = 0.0, v_threshold: float = 1.0, v_reset: Optional[float] = 0.0,
                 surrogate_function=surrogate.Rect()):
        self.act_dim, self.dec_pop_dim = act_dim, dec_pop_dim
        super().__init__(act_dim * dec_pop_dim, is_training, T, sigma_init, beta, v_threshold, v_reset,
                         surrogate_function)
        self.conn = nn.Conv1d(act_dim, self.num_node, dec_pop_dim, groups=act_dim)

    def _after_spike(self, t, spike):
        if t + 1 == self.T:
            return None
        return self.conn(spike.view(-1, self.act_dim, self.dec_pop_dim)).view(-1, self.num_node)


class NoisyILCCUBALIFNode(_CubaCharge, NoisyILCBaseNode):
    def __init__(self, act_dim, dec_pop_dim, c_decay: float = 0.5, v_decay: float = 0.75, is_training: bool = True,
                 T: int = 5, sigma_init: float = 0.5, beta: float = 0.0, v_threshold: float = 1.0,
                 v_reset: Optional[float] = 0.0, surrogate_function=surrogate.Rect()):
        super().__init__(act_dim, dec_pop_dim, is_training, T, sigma_init, beta, v_threshold, v_reset,
                         surrogate_function)
        self.c_decay, self.v_decay = c_decay, v_decay


class NoisyNonSpikingBaseNode(nn.Module, base.MultiStepModule):
    """Non-spiking read-out with learnable per-neuron noise scale ``sigma`` (a parameter)."""

    def __init__(self, num_node, is_training: bool = True, T: int = 5, sigma_init: float = 0.5, beta: float = 0.0,
                 decode: Optional[str] = None):
        super().__init__()
        self.num_node, self.is_training, self.T, self.beta, self.decode = num_node, is_training, T, beta, decode
        self.sigma = nn.Parameter(torch.full((num_node,), sigma_init / math.sqrt(num_node), dtype=torch.float))
        self.cn = None

    @abstractmethod
    def neuronal_charge(self, x):
        raise NotImplementedError

    def init_tensor(self, data):
        self.v = torch.zeros_like(data)

    def forward(self, x_seq):
        self.init_tensor(x_seq[0])
        if self.is_training and self.cn is None:
            self.noise_step += 1
        trace = []
        for t in range(self.T):
            x = x_seq[t]
            if self.is_training:
                noise = (self.eps_seq[self.noise_step][t] if self.cn is None else self.cn[:, t]).to(x_seq.device)
                x = x + self.sigma * noise
            self.neuronal_charge(x)
            trace.append(self.v)
        if self.decode not in {"max-mem", "max-abs-mem", "mean-mem", "last-me"}:
            return trace
        stack = torch.stack(trace)
        if self.decode == "max-mem":
            return stack.max(0).values
        if self.decode == "max-abs-mem":
            hi, lo = stack.max(0).values, stack.min(0).values
            return torch.where(hi.abs() > lo.abs(), hi, lo)
        if self.decode == "mean-mem":
            return stack.mean(0)
        return trace[-1]

    def reset_noise(self, num_rl_step):
        self.eps_seq = _noise_table(self.beta, self.num_node, num_rl_step, self.T)
        self.noise_step = -1

    def get_colored_noise(self):
        return self.eps_seq[self.noise_step]

    def load_colored_noise(self, cn):
        self.cn = cn

    def cancel_load(self):
        self.cn = None


class NoisyNonSpikingIFNode(NoisyNonSpikingBaseNode):
    def neuronal_charge(self, x):
        self.v = self.v + x
