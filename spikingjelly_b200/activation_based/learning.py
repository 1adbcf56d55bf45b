"""Spike-timing-dependent plasticity learners (STDP, reward-modulated MSTDP and MSTDPET).

A learner watches one synapse (``nn.Linear`` / ``nn.Conv1d`` / ``nn.Conv2d``) and the neuron layer
behind it through monitors, keeps the pre / post traces as module memories, and on ``step()``
consumes everything recorded since the last call and either subtracts the weight change from
``synapse.weight.grad`` (so that any optimiser *ascends* it) or returns it.

The per-step math lives in :mod:`~spikingjelly_b200.activation_based.functional.learning`.
Parity: ``spikingjelly/activation_based/learning.py:42-1434``.
"""
from __future__ import annotations

from typing import Callable, Optional, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import base, monitor, neuron
from .functional import learning as FL

__all__ = ["stdp_linear_single_step", "mstdp_linear_single_step", "mstdpet_linear_single_step", "stdp_conv2d_single_step",
           "stdp_conv1d_single_step", "stdp_multi_step", "STDPLearner", "MSTDPLearner", "MSTDPETLearner"]


def _identity(x):
    return x


def _trace_tensor(trace, like: torch.Tensor) -> torch.Tensor:
    if isinstance(trace, torch.Tensor):
        return trace
    return torch.full_like(like, 0.0 if trace is None else trace)


def _pad_like_conv(conv, x: torch.Tensor) -> torch.Tensor:
    """The input as the convolution sees it (its padding applied explicitly)."""
    if not any(conv.padding):
        return x
    if conv.padding_mode != "zeros":
        return F.pad(x, conv._reversed_padding_repeated_twice, mode=conv.padding_mode)
    pads = []
    for p in reversed(conv.padding):
        pads += [p, p]
    return F.pad(x, tuple(pads))


def _accumulate_weight_gradient(synapse, delta_w) -> None:
    synapse.weight.grad = -delta_w if synapse.weight.grad is None else synapse.weight.grad - delta_w


def _linear_rule(step_fn):
    def single_step(fc: nn.Linear, in_spike, out_spike, trace_pre, trace_post, tau_pre: float, tau_post: float,
                    f_pre: Callable = _identity, f_post: Callable = _identity):
        out, (trace_pre, trace_post) = step_fn(in_spike, out_spike,
                                               (_trace_tensor(trace_pre, in_spike), _trace_tensor(trace_post, out_spike)),
                                               fc.weight.data, tau_pre=tau_pre, tau_post=tau_post, f_pre=f_pre, f_post=f_post)
        return trace_pre, trace_post, out
    return single_step


stdp_linear_single_step = _linear_rule(FL.stdp_linear_step)
stdp_linear_single_step.__name__ = "stdp_linear_single_step"
stdp_linear_single_step.__doc__ = """One STDP step of a fully connected synapse.
``in_spike [B, N_in]``, ``out_spike [B, N_out]`` -> ``(trace_pre, trace_post, delta_w [N_out, N_in])`` with
``trace <- trace - trace / tau + spike`` and ``delta_w = f_post(w) * outer(out_spike, trace_pre) - f_pre(w) * outer(trace_post, in_spike)``
summed over the batch."""
mstdp_linear_single_step = _linear_rule(FL.mstdp_linear_step)
mstdp_linear_single_step.__name__ = "mstdp_linear_single_step"
mstdp_linear_single_step.__doc__ = """As ``stdp_linear_single_step`` but returns the per-sample eligibility ``[B, N_out, N_in]`` (not summed)."""
mstdpet_linear_single_step = _linear_rule(FL.mstdpet_linear_step)
mstdpet_linear_single_step.__name__ = "mstdpet_linear_single_step"
mstdpet_linear_single_step.__doc__ = """As ``stdp_linear_single_step`` but returns the batch-summed eligibility fed to the eligibility trace."""


def _conv_rule(step_fn, cls, dilation_one):
    def single_step(conv, in_spike, out_spike, trace_pre, trace_post, tau_pre: float, tau_post: float,
                    f_pre: Callable = _identity, f_post: Callable = _identity):
        if conv.dilation != dilation_one:
            raise NotImplementedError(f"STDP with dilation != 1 for {cls.__name__} has not been implemented!")
        if conv.groups != 1:
            raise NotImplementedError(f"STDP with groups != 1 for {cls.__name__} has not been implemented!")
        in_spike = _pad_like_conv(conv, in_spike)
        traces = (torch.zeros_like(in_spike) if trace_pre is None else trace_pre,
                  torch.zeros_like(out_spike) if trace_post is None else trace_post)
        delta_w, (trace_pre, trace_post) = step_fn(in_spike, out_spike, traces, conv.weight.data, stride=conv.stride,
                                                   tau_pre=tau_pre, tau_post=tau_post, f_pre=f_pre, f_post=f_post)
        return trace_pre, trace_post, delta_w
    return single_step


stdp_conv2d_single_step = _conv_rule(FL.stdp_conv2d_step, nn.Conv2d, (1, 1))
stdp_conv2d_single_step.__name__ = "stdp_conv2d_single_step"
stdp_conv2d_single_step.__doc__ = """One STDP step of a 2-D convolution (``groups == 1``, ``dilation == 1``); the pre-synaptic trace lives on the padded input."""
stdp_conv1d_single_step = _conv_rule(FL.stdp_conv1d_step, nn.Conv1d, (1,))
stdp_conv1d_single_step.__name__ = "stdp_conv1d_single_step"
stdp_conv1d_single_step.__doc__ = """One STDP step of a 1-D convolution (``groups == 1``, ``dilation == 1``)."""


def _single_step_rule(layer):
    if isinstance(layer, nn.Linear):
        return stdp_linear_single_step
    if isinstance(layer, nn.Conv1d):
        return stdp_conv1d_single_step
    if isinstance(layer, nn.Conv2d):
        return stdp_conv2d_single_step
    raise NotImplementedError(layer)


def stdp_multi_step(layer, in_spike, out_spike, trace_pre, trace_post, tau_pre: float, tau_post: float,
                    f_pre: Callable = _identity, f_post: Callable = _identity):
    """STDP over a sequence ``[T, B, ...]``: the traces are carried through time, the weight changes summed."""
    if in_spike.shape[0] == 0:
        return trace_pre, trace_post, torch.zeros_like(layer.weight)
    rule = _single_step_rule(layer)
    delta_w = torch.zeros_like(layer.weight)
    for t in range(in_spike.shape[0]):
        trace_pre, trace_post, dw = rule(layer, in_spike[t], out_spike[t], trace_pre, trace_post, tau_pre, tau_post, f_pre, f_post)
        delta_w += dw
    return trace_pre, trace_post, delta_w


class _Learner(base.MemoryModule):
    """Monitors, traces, enable / disable / reset shared by the three learners."""

    def __init__(self, step_mode: str, synapse, sn: neuron.BaseNode, tau_pre: float, tau_post: float, f_pre: Callable,
                 f_post: Callable):
        super().__init__()
        self.step_mode = step_mode
        self.tau_pre, self.tau_post = tau_pre, tau_post
        self.f_pre, self.f_post = f_pre, f_post
        self.synapse = synapse
        self.in_spike_monitor = monitor.InputMonitor(synapse, function_on_input=torch.Tensor.detach)
        self.out_spike_monitor = monitor.OutputMonitor(sn, function_on_output=torch.Tensor.detach)
        self.register_memory("trace_pre", None)
        self.register_memory("trace_post", None)

    def reset(self):
        """Forget traces (and eligibilities) and drop the spikes recorded so far."""
        super().reset()
        self.in_spike_monitor.clear_recorded_data()
        self.out_spike_monitor.clear_recorded_data()

    def disable(self):
        """Stop recording spikes (e.g. during evaluation)."""
        self.in_spike_monitor.disable()
        self.out_spike_monitor.disable()

    def enable(self):
        self.in_spike_monitor.enable()
        self.out_spike_monitor.enable()

    def _recorded(self):
        for _ in range(len(self.in_spike_monitor.records)):
            yield self.in_spike_monitor.records.pop(0), self.out_spike_monitor.records.pop(0)

    def _reward_rule(self, rule):
        """The reward-modulated learners only exist for single-step fully connected synapses."""
        if self.step_mode == "s":
            if isinstance(self.synapse, nn.Linear):
                return rule
            raise NotImplementedError(self.synapse)
        if self.step_mode == "m":
            raise NotImplementedError(self.synapse)
        raise ValueError(self.step_mode)

    def _finish(self, delta_w, on_grad: bool):
        if on_grad:
            _accumulate_weight_gradient(self.synapse, delta_w)
            return None
        return delta_w


class STDPLearner(_Learner):
    """Pair-based STDP with exponential traces for ``nn.Linear`` / ``nn.Conv1d`` / ``nn.Conv2d``
    (single- or multi-step records).  ``step(on_grad=True, scale=1.0)``."""

    def __init__(self, step_mode: str, synapse: Union[nn.Conv2d, nn.Linear], sn: neuron.BaseNode, tau_pre: float,
                 tau_post: float, f_pre: Callable = _identity, f_post: Callable = _identity):
        super().__init__(step_mode, synapse, sn, tau_pre, tau_post, f_pre, f_post)

    def step(self, on_grad: bool = True, scale: float = 1.0):
        if self.step_mode == "s":
            rule = _single_step_rule(self.synapse)
        elif self.step_mode == "m":
            if not isinstance(self.synapse, (nn.Linear, nn.Conv1d, nn.Conv2d)):
                raise NotImplementedError(self.synapse)
            rule = stdp_multi_step
        else:
            raise ValueError(self.step_mode)
        delta_w = None
        for in_spike, out_spike in self._recorded():
            self.trace_pre, self.trace_post, dw = rule(self.synapse, in_spike, out_spike, self.trace_pre, self.trace_post,
                                                       self.tau_pre, self.tau_post, self.f_pre, self.f_post)
            if scale != 1.0:
                dw *= scale
            delta_w = dw if delta_w is None else delta_w + dw
        return self._finish(delta_w, on_grad)


class MSTDPLearner(_Learner):
    """Reward-modulated STDP (Florian 2007): ``delta_w = sum_b reward_b * eligibility_b`` where the
    eligibility is the per-sample STDP update of the *previous* step.  ``reward``: ``[batch_size]``."""

    def __init__(self, step_mode: str, batch_size: float, synapse: Union[nn.Conv2d, nn.Linear], sn: neuron.BaseNode,
                 tau_pre: float, tau_post: float, f_pre: Callable = _identity, f_post: Callable = _identity):
        super().__init__(step_mode, synapse, sn, tau_pre, tau_post, f_pre, f_post)
        self.batch_size = batch_size
        self.register_memory("eligibility", None)

    def step(self, reward, on_grad: bool = True, scale: float = 1.0):
        if isinstance(reward, torch.Tensor):
            reward = reward.detach()        # a reward computed by a network must not drag its graph into weight.grad
        rule = self._reward_rule(mstdp_linear_single_step)
        delta_w = None
        for in_spike, out_spike in self._recorded():
            if self.eligibility is None:
                self.eligibility = torch.zeros(self.batch_size, *self.synapse.weight.shape, device=self.synapse.weight.device)
            dw = (reward.view(-1, 1, 1) * self.eligibility).sum(0)
            if scale != 1.0:
                dw *= scale
            delta_w = dw if delta_w is None else delta_w + dw
            self.trace_pre, self.trace_post, self.eligibility = rule(self.synapse, in_spike, out_spike, self.trace_pre,
                                                                     self.trace_post, self.tau_pre, self.tau_post, self.f_pre,
                                                                     self.f_post)
        return self._finish(delta_w, on_grad)


class MSTDPETLearner(_Learner):
    """Reward-modulated STDP with an eligibility trace of time constant ``tau_trace``
    (``trace_e <- trace_e * exp(-1/tau_trace) + eligibility / tau_trace``, ``delta_w = reward * trace_e``)."""

    def __init__(self, step_mode: str, synapse: Union[nn.Conv2d, nn.Linear], sn: neuron.BaseNode, tau_pre: float,
                 tau_post: float, tau_trace: float, f_pre: Callable = _identity, f_post: Callable = _identity):
        super().__init__(step_mode, synapse, sn, tau_pre, tau_post, f_pre, f_post)
        self.tau_trace = tau_trace
        self.register_memory("trace_e", None)
        self.register_memory("eligibility", None)

    def step(self, reward, on_grad: bool = True, scale: float = 1.0):
        if isinstance(reward, torch.Tensor):
            reward = reward.detach()
        rule = self._reward_rule(mstdpet_linear_single_step)
        delta_w = None
        for in_spike, out_spike in self._recorded():
            if self.eligibility is None:
                self.eligibility = torch.zeros_like(self.synapse.weight)
            if self.trace_e is None:
                self.trace_e = torch.zeros_like(self.synapse.weight)
            dw, self.trace_e = FL.mstdpet_reward_step(reward, self.eligibility, self.trace_e, tau_trace=self.tau_trace)
            if scale != 1.0:
                dw *= scale
            delta_w = dw if delta_w is None else delta_w + dw
            self.trace_pre, self.trace_post, self.eligibility = rule(self.synapse, in_spike, out_spike, self.trace_pre,
                                                                     self.trace_post, self.tau_pre, self.tau_post, self.f_pre,
                                                                     self.f_post)
        return self._finish(delta_w, on_grad)
