"""Quadratic and exponential integrate-and-fire neurons (``neuron/nonlinear_if.py:12-473``)
and the two-state Izhikevich neuron (``neuron/adapt.py:12-399``)."""
from __future__ import annotations

from typing import Optional

import weakref

import torch

from .. import functional, surrogate
from .base_node import BaseNode

__all__ = ["QIFNode", "EIFNode", "AdaptBaseNode", "IzhikevichNode"]


class QIFNode(BaseNode):
    """``h = v + (x + a0 (v - v_rest)(v - v_c)) / tau``."""
    _has_native = True

    def __init__(self, tau: float = 2.0, v_c: float = 0.8, a0: float = 1.0, v_threshold: float = 1.0,
                 v_rest: float = 0.0, v_reset: Optional[float] = -0.1, surrogate_function=surrogate.Sigmoid(),
                 detach_reset: bool = False, step_mode="s", backend="torch", store_v_seq: bool = False):
        assert isinstance(tau, float) and tau > 1.0
        if v_reset is not None:
            assert v_threshold > v_reset
            assert v_rest >= v_reset
        assert a0 > 0
        super().__init__(v_threshold, v_reset, surrogate_function, detach_reset, step_mode, backend, store_v_seq)
        self.tau, self.v_c, self.v_rest, self.a0 = tau, v_c, v_rest, a0

    def extra_repr(self):
        return super().extra_repr() + f", tau={self.tau}, v_c={self.v_c}, a0={self.a0}, v_rest={self.v_rest}"

    def _eager_step(self, x, v, sg):
        return functional.qif_step(x, v, self.tau, self.a0, self.v_rest, self.v_c, self.v_threshold, self.v_reset, sg,
                                   self.detach_reset)

    def _native_sequence(self, x_seq, v, store_v_seq):
        return functional.qif_multi_step_cuda(x_seq, v, self.tau, self.v_c, self.a0, self.v_threshold, self.v_rest,
                                              self.v_reset, self.surrogate_function, self.detach_reset, store_v_seq)


class EIFNode(BaseNode):
    """``h = v + (x + v_rest - v + delta_T exp((v - theta_rh)/delta_T)) / tau``."""
    _has_native = True

    def __init__(self, tau: float = 2.0, delta_T: float = 1.0, theta_rh: float = 0.8, v_threshold: float = 1.0,
                 v_rest: float = 0.0, v_reset: Optional[float] = -0.1, surrogate_function=surrogate.Sigmoid(),
                 detach_reset: bool = False, step_mode="s", backend="torch", store_v_seq: bool = False):
        assert isinstance(tau, float) and tau > 1.0
        if v_reset is not None:
            assert v_threshold > v_reset
            assert v_rest >= v_reset
        assert delta_T > 0
        super().__init__(v_threshold, v_reset, surrogate_function, detach_reset, step_mode, backend, store_v_seq)
        self.tau, self.delta_T, self.v_rest, self.theta_rh = tau, delta_T, v_rest, theta_rh

    def extra_repr(self):
        return (super().extra_repr() + f", tau={self.tau}, delta_T={self.delta_T}, theta_rh={self.theta_rh}")

    def _eager_step(self, x, v, sg):
        return functional.eif_step(x, v, self.tau, self.delta_T, self.theta_rh, self.v_rest, self.v_threshold,
                                   self.v_reset, sg, self.detach_reset)

    def _native_sequence(self, x_seq, v, store_v_seq):
        return functional.eif_multi_step_cuda(x_seq, v, self.tau, self.v_threshold, self.v_reset, self.v_rest,
                                              self.theta_rh, self.delta_T, self.surrogate_function, self.detach_reset,
                                              store_v_seq)


class AdaptBaseNode(BaseNode):
    """Base of neurons with an adaptation current ``w`` (second memory)."""

    def __init__(self, v_threshold: float = 1.0, v_reset: Optional[float] = 0.0, v_rest: float = 0.0,
                 w_rest: float = 0.0, tau_w: float = 2.0, a: float = 0.0, b: float = 0.0,
                 surrogate_function=surrogate.Sigmoid(), detach_reset: bool = False, step_mode="s", backend="torch",
                 store_v_seq: bool = False):
        for val in (w_rest, v_rest, tau_w, a, b):
            assert isinstance(val, float)
        super().__init__(v_threshold, v_reset, surrogate_function, detach_reset, step_mode, backend, store_v_seq)
        self.register_memory("w", w_rest)
        self.w_rest, self.v_rest, self.tau_w, self.a, self.b = w_rest, v_rest, tau_w, a, b

    @staticmethod
    def jit_neuronal_adaptation(w, tau_w: float, a: float, v_rest: float, v):
        return w + 1.0 / tau_w * (a * (v - v_rest) - w)

    def neuronal_adaptation(self):
        self.w = self.jit_neuronal_adaptation(self.w, self.tau_w, self.a, self.v_rest, self.v)

    def extra_repr(self):
        return (super().extra_repr() + f", v_rest={self.v_rest}, w_rest={self.w_rest}, tau_w={self.tau_w}, "
                f"a={self.a}, b={self.b}")

    def materialize_states(self, inputs, states, step_mode):
        states = super().materialize_states(inputs, states, step_mode)
        ref, w = states[0], states[-1]
        if isinstance(w, float):
            w = torch.full_like(ref, w, requires_grad=False)
        elif isinstance(w, torch.Tensor):
            if w.shape != ref.shape:
                w = torch.full_like(ref, self.w_rest, requires_grad=False)
            elif w.dtype != ref.dtype or w.device != ref.device:
                w = w.to(dtype=ref.dtype, device=ref.device)
        return (*states[:-1], w)


class IzhikevichNode(AdaptBaseNode):
    def __init__(self, tau: float = 2.0, v_c: float = 0.8, a0: float = 1.0, v_threshold: float = 1.0,
                 v_reset: Optional[float] = 0.0, v_rest: float = -0.1, w_rest: float = 0.0, tau_w: float = 2.0,
                 a: float = 0.0, b: float = 0.0, surrogate_function=surrogate.Sigmoid(), detach_reset: bool = False,
                 step_mode="s", backend="torch", store_v_seq: bool = False):
        assert isinstance(tau, float) and tau > 1.0
        assert a0 > 0
        super().__init__(v_threshold, v_reset, v_rest, w_rest, tau_w, a, b, surrogate_function, detach_reset,
                         step_mode, backend, store_v_seq)
        self.tau, self.v_c, self.a0 = tau, v_c, a0

    @property
    def supported_backends(self):
        return ("torch",) if self.step_mode == "s" else ("torch", "cuda", "cupy")

    def extra_repr(self):
        return super().extra_repr() + f", tau={self.tau}, v_c={self.v_c}, a0={self.a0}"

    def single_step_functional_forward(self, inputs, states, **kwargs):
        spike, v, w = functional.izhikevich_step(
            inputs[0], states[0], states[-1], self.tau, self.a0, self.v_rest, self.v_c, self.tau_w, self.a, self.b,
            self.v_threshold, self.v_reset, self.surrogate_function, self.detach_reset)
        return (spike,), (v, w)

    def _compiled(self):
        from ._compiled import CompiledSequence, compiled_for, scalar_signature
        ref = weakref.ref(self)

        def step(x, v, w):
            (spike,), (v2, w2) = ref().single_step_functional_forward((x,), (v, w))
            return spike, v2, w2

        return compiled_for(self, lambda: CompiledSequence(step, 2, lambda: scalar_signature(ref()), "izhikevich"))

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        if self.native and inputs[0].is_cuda and getattr(self.surrogate_function, "spiking", True):
            res = self._compiled().run(inputs[0], (states[0], states[-1]))
            if res is not None:
                spike_seq, (v, w), _ = res
                return (spike_seq,), (v, w)
        return super(BaseNode, self).multi_step_functional_forward(inputs, states, **kwargs)
