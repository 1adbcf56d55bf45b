"""Leaky integrate-and-fire neurons.

Parity: ``neuron/lif.py`` — ``SimpleLIFNode`` :12-94, ``LIFNode`` :97-398,
``NonSpikingLIFNode`` :401-421; ``neuron/plif.py:14-261`` (``ParametricLIFNode``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import functional, surrogate
from .base_node import BaseNode, NonSpikingBaseNode, SimpleBaseNode

__all__ = ["SimpleLIFNode", "LIFNode", "NonSpikingLIFNode", "ParametricLIFNode"]


class SimpleLIFNode(SimpleBaseNode):
    def __init__(self, tau: float, decay_input: bool, v_threshold: float = 1.0, v_reset: float = 0.0,
                 surrogate_function=surrogate.Sigmoid(), detach_reset: bool = False, step_mode="s"):
        super().__init__(v_threshold, v_reset, surrogate_function, detach_reset, step_mode)
        self.tau = tau
        self.decay_input = decay_input

    def neuronal_charge(self, x):
        leak = self.v_reset - self.v
        self.v = self.v + ((leak + x) / self.tau if self.decay_input else leak / self.tau + x)


class LIFNode(BaseNode):
    """``decay_input``: ``h = v + (x - (v - v_reset)) / tau``; else ``h = v - (v - v_reset) / tau + x``."""
    _has_native = True
    _native_single_step = True

    def __init__(self, tau: float = 2.0, decay_input: bool = True, v_threshold: float = 1.0,
                 v_reset: Optional[float] = 0.0, surrogate_function=surrogate.Sigmoid(), detach_reset: bool = False,
                 step_mode="s", backend="torch", store_v_seq: bool = False):
        assert isinstance(tau, float) and tau > 1.0
        super().__init__(v_threshold, v_reset, surrogate_function, detach_reset, step_mode, backend, store_v_seq)
        self.tau = tau
        self.decay_input = decay_input

    def extra_repr(self):
        return super().extra_repr() + f", tau={self.tau}"

    def _eager_step(self, x, v, sg):
        return functional.lif_step(x, v, self.tau, self.decay_input, self.v_threshold, self.v_reset, sg,
                                   self.detach_reset)

    def _native_sequence(self, x_seq, v, store_v_seq):
        return functional.lif_multi_step_cuda(x_seq, v, self.tau, self.decay_input, self.v_threshold, self.v_reset,
                                              self.surrogate_function, self.detach_reset, store_v_seq)


class NonSpikingLIFNode(NonSpikingBaseNode):
    def __init__(self, tau: float = 2.0, decode: Optional[str] = None):
        super().__init__(decode)
        self.tau = tau

    def neuronal_charge(self, x):
        self.v = self.v + (x - self.v) / self.tau


class ParametricLIFNode(BaseNode):
    """LIF whose ``1/tau = sigmoid(w)`` is learned; ``w`` is a 0-dim parameter initialised
    to ``-log(init_tau - 1)`` (the only ``state_dict`` key of the neuron)."""
    _has_native = True

    def __init__(self, init_tau: float = 2.0, decay_input: bool = True, v_threshold: float = 1.0,
                 v_reset: Optional[float] = 0.0, surrogate_function=surrogate.Sigmoid(), detach_reset: bool = False,
                 step_mode="s", backend="torch", store_v_seq: bool = False):
        assert isinstance(init_tau, float) and init_tau > 1.0
        super().__init__(v_threshold, v_reset, surrogate_function, detach_reset, step_mode, backend, store_v_seq)
        self.decay_input = decay_input
        self.w = nn.Parameter(torch.as_tensor(-math.log(init_tau - 1.0)))

    def extra_repr(self):
        with torch.no_grad():
            tau = 1.0 / self.w.sigmoid()
        return super().extra_repr() + f", tau={tau}"

    def _eager_step(self, x, v, sg):
        return functional.plif_step(x, v, self.w, self.decay_input, self.v_threshold, self.v_reset, sg,
                                    self.detach_reset)

    def _native_sequence(self, x_seq, v, store_v_seq):
        return functional.plif_multi_step_cuda(x_seq, v, self.w.sigmoid(), self.decay_input, self.v_threshold,
                                               self.v_reset, self.surrogate_function, self.detach_reset, store_v_seq)
