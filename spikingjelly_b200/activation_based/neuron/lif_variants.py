"""LIF variants: gated (GLIF), k-scaled (KLIF), current-based (CUBA), analog-output (LIAF),
integer-spike (ILIF).

Parity: ``neuron/lif_variants.py:15-660`` and ``neuron/ilif.py:17-410``.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import numpy as np
import weakref

import torch
import torch.nn as nn

from .. import base, functional, surrogate
from .base_node import BaseNode
from .lif import LIFNode

__all__ = ["GatedLIFNode", "KLIFNode", "CUBALIFNode", "LIAFNode", "ILIFNode"]


def _logit(p: float) -> float:
    return -math.log(1.0 / p - 1.0)


class GatedLIFNode(base.MemoryModule):
    """GLIF: learnable gates (sigmoid of ``alpha, beta, gamma``) mix two variants of each of
    leak, reset and input integration; ``tau, v_threshold, linear_decay, v_subreset`` and the
    per-step ``conduct`` are learnable as well (all stored as logits).  Multi-step only;
    channel-wise when ``inplane`` is given (input ``[T, N, C, H, W]``)."""

    def __init__(self, T: int, inplane=None, init_linear_decay=None, init_v_subreset=None, init_tau: float = 0.25,
                 init_v_threshold: float = 0.5, init_conduct: float = 0.5, surrogate_function=surrogate.Sigmoid(),
                 step_mode="m", backend="torch"):
        assert isinstance(init_tau, float) and init_tau < 1.0
        assert isinstance(T, int) and T is not None
        assert isinstance(inplane, int) or inplane is None
        assert (isinstance(init_linear_decay, float) and init_linear_decay < 1.0) or init_linear_decay is None
        assert (isinstance(init_v_subreset, float) and init_v_subreset < 1.0) or init_v_subreset is None
        assert step_mode == "m"
        super().__init__()
        self.surrogate_function = surrogate_function
        self.backend = backend
        self.step_mode = step_mode
        self.T = T
        self.register_memory("v", 0.0)
        self.register_memory("u", 0.0)
        shape = () if inplane is None else (inplane,)
        for name in ("alpha", "beta", "gamma"):
            setattr(self, name, nn.Parameter(torch.tensor(0.2 * (np.random.rand(*shape) - 0.5), dtype=torch.float)))
        if init_linear_decay is None:
            init_linear_decay = init_v_threshold / (T * 2)
        if init_v_subreset is None:
            init_v_subreset = init_v_threshold
        self.tau = nn.Parameter(torch.full(shape, _logit(init_tau), dtype=torch.float))
        self.v_threshold = nn.Parameter(torch.full(shape, _logit(init_v_threshold), dtype=torch.float))
        self.linear_decay = nn.Parameter(torch.full(shape, _logit(init_linear_decay), dtype=torch.float))
        self.v_subreset = nn.Parameter(torch.full(shape, _logit(init_v_subreset), dtype=torch.float))
        self.conduct = nn.Parameter(torch.full((T, *shape), _logit(init_conduct), dtype=torch.float))

    @property
    def supported_backends(self):
        return ("torch",)

    def extra_repr(self):
        return (super().extra_repr() + f", tau={self.tau}, v_subreset={self.v_subreset}, "
                f"linear_decay={self.linear_decay}, conduct={self.conduct}")

    def materialize_states(self, inputs, states, step_mode):
        v = states[0]
        if not isinstance(v, torch.Tensor):
            v = torch.full_like(inputs[0][0], v)
        return v, states[1]

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        x_seq, v = inputs[0], states[0]
        gate = lambda p: p.view(1, -1, 1, 1).sigmoid()  # noqa: E731
        alpha, beta, gamma = gate(self.alpha), gate(self.beta), gate(self.gamma)
        tau, v_th = gate(self.tau), gate(self.v_threshold)
        decay, subreset = gate(self.linear_decay), gate(self.v_subreset)
        spike = torch.zeros(x_seq.shape[1:], device=x_seq.device)
        out = []
        for t in range(self.T):
            spike, v = functional.gated_lif_step(x_seq[t], v, spike, alpha, beta, gamma, tau, v_th, decay, subreset,
                                                 gate(self.conduct[t]), self.surrogate_function)
            out.append(spike)
        return (torch.stack(out),), (v, v)


class KLIFNode(BaseNode):
    """LIF whose charged potential passes through ``relu(k * h)`` with learnable ``k``."""

    def __init__(self, scale_reset: bool = False, tau: float = 2.0, decay_input: bool = True, v_threshold: float = 1.0,
                 v_reset: Optional[float] = 0.0, surrogate_function=surrogate.Sigmoid(), detach_reset: bool = False,
                 step_mode="s", backend="torch", store_v_seq: bool = False):
        assert isinstance(tau, float) and tau > 1.0
        super().__init__(v_threshold, v_reset, surrogate_function, detach_reset, step_mode, backend, store_v_seq)
        self.scale_reset, self.tau, self.decay_input = scale_reset, tau, decay_input
        self.k = nn.Parameter(torch.as_tensor(1.0))

    def _eager_surrogate(self):
        return self.surrogate_function

    def _eager_step(self, x, v, sg):
        return functional.klif_step(x, v, self.k, self.tau, self.decay_input, self.scale_reset, self.v_threshold,
                                    self.v_reset, sg, self.detach_reset)


class CUBALIFNode(BaseNode):
    """Current-based LIF: ``c <- c * c_decay + x``; ``h = v * v_decay + c``."""

    def __init__(self, c_decay: float = 0.5, v_decay: float = 0.75, v_threshold: float = 0.5,
                 v_reset: Optional[float] = 0.0, surrogate_function=surrogate.Rect()):
        super().__init__(v_threshold, v_reset, surrogate_function)
        self.register_memory("c", 0.0)
        self.c_decay, self.v_decay = c_decay, v_decay

    def materialize_states(self, inputs, states, step_mode):
        states = super().materialize_states(inputs, states, step_mode)
        ref, c = states[0], states[1]
        if isinstance(c, float):
            c = torch.full_like(ref, c, requires_grad=False)
        elif isinstance(c, torch.Tensor):
            if c.shape != ref.shape:
                c = torch.zeros_like(ref, requires_grad=False)
            elif c.dtype != ref.dtype or c.device != ref.device:
                c = c.to(dtype=ref.dtype, device=ref.device)
        return (states[0], c, *states[2:])

    def single_step_functional_forward(self, inputs, states, **kwargs):
        v, c = states
        spike, c, v = functional.cuba_lif_step(inputs[0], c, v, self.c_decay, self.v_decay, self.v_threshold,
                                               self.v_reset, self.surrogate_function, self.detach_reset)
        return (spike,), (v, c)


class LIAFNode(LIFNode):
    """LIF dynamics, analog output ``act(h)`` (or ``act(h - v_th)`` when ``threshold_related``)."""
    _has_native = False

    def __init__(self, act: Callable, threshold_related: bool, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.act, self.threshold_related = act, threshold_related
        assert self.backend == "torch", "LIAFNode only supports for backend='torch'!"

    def single_step_functional_forward(self, inputs, states, **kwargs):
        y, v = functional.liaf_step(inputs[0], states[0], self.tau, self.decay_input, self.v_threshold, self.v_reset,
                                    self.act, self.threshold_related, self.surrogate_function, self.detach_reset)
        return (y,), (v, *states[1:])


class ILIFNode(LIFNode):
    """Integer-valued LIF: emits ``round(clamp(h / v_th, 0, D))`` spikes per step and subtracts
    ``spikes * v_th`` (soft reset); the input is not decayed.  Default ``tau = 4/3``."""
    _has_native = False

    def __init__(self, tau: float = 4.0 / 3.0, v_threshold: float = 1.0,
                 surrogate_function=surrogate.MultiLevelSpikeCount(4), detach_reset: bool = False,
                 step_mode: str = "s", backend: str = "torch", store_v_seq: bool = False) -> None:
        if not isinstance(surrogate_function, surrogate.MultiLevelSpikeCount) or not surrogate_function.spiking:
            raise ValueError("surrogate_function must be a spiking MultiLevelSpikeCount.")
        super().__init__(tau=tau, decay_input=False, v_threshold=v_threshold, v_reset=None,
                         surrogate_function=surrogate_function, detach_reset=detach_reset, step_mode=step_mode,
                         backend="torch", store_v_seq=store_v_seq)
        self._backend = backend if backend in self.supported_backends else "torch"

    @property
    def supported_backends(self):
        return ("torch",) if self.step_mode == "s" else ("torch", "cuda", "triton")

    def _use_native(self, x):
        return False      # integer spikes: the eager rule runs on every device

    def _eager_surrogate(self):
        return self.surrogate_function

    def _eager_step(self, x, v, sg):
        return functional.ilif_step(x, v, self.tau, self.v_threshold, sg, self.detach_reset)

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        if self.native and inputs[0].is_cuda:
            from ._compiled import CompiledSequence, compiled_for, scalar_signature
            ref = weakref.ref(self)

            def step(x, v):
                me = ref()
                return me._eager_step(x, v, me.surrogate_function)

            seq = compiled_for(self, lambda: CompiledSequence(step, 1, lambda: scalar_signature(ref()), "ilif"))
            res = seq.run(inputs[0], (states[0],))
            if res is not None:
                return (res[0],), (res[1][0], *states[1:])
        return super().multi_step_functional_forward(inputs, states, **kwargs)
