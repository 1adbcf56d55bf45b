"""Neuron base classes.

``BaseNode`` owns the membrane potential ``v`` (a memory), the step-mode/backend
dispatch and ``store_v_seq``.  A concrete neuron only describes its dynamics:

* ``_eager_step(x, v, sg) -> (spike, v_next)`` — PyTorch ops, any device (oracle);
* ``_native_sequence(x_seq, v, store_v_seq) -> (spike_seq, v_last, v_seq)`` —
  optional: the whole sequence in one sm_100a kernel.

Parity: ``spikingjelly/activation_based/neuron/base_node.py`` — ``SimpleBaseNode``
:12-249, ``BaseNode`` :252-485, ``NonSpikingBaseNode`` :488-526.
"""
from __future__ import annotations

from abc import abstractmethod
from typing import Optional

import torch
import torch.nn as nn

from .. import base, surrogate

__all__ = ["BaseNode", "NonSpikingBaseNode", "SimpleBaseNode"]

_ALL_BACKENDS = ("torch", "cuda", "cupy", "triton", "inductor")


class SimpleBaseNode(base.MemoryModule):
    """Minimal neuron written as three overridable hooks (charge, fire, reset) acting on
    ``self.v``; multi-step mode is a Python loop.  Meant for teaching and prototyping."""

    def __init__(self, v_threshold: float = 1.0, v_reset: Optional[float] = 0.0,
                 surrogate_function: surrogate.SurrogateFunctionBase = surrogate.Sigmoid(),
                 detach_reset: bool = False, step_mode="s"):
        super().__init__()
        self.v_threshold = v_threshold
        self.v_reset = v_reset
        self.surrogate_function = surrogate_function
        self.detach_reset = detach_reset
        self.step_mode = step_mode
        self.register_memory("v", 0.0)

    def neuronal_charge(self, x: torch.Tensor) -> None:
        raise NotImplementedError

    def neuronal_fire(self) -> torch.Tensor:
        return self.surrogate_function(self.v - self.v_threshold)

    def neuronal_reset(self, spike: torch.Tensor) -> None:
        s = spike.detach() if self.detach_reset else spike
        if self.v_reset is None:
            self.v = self.v - self.v_threshold * s
        else:
            self.v = s * self.v_reset + (1.0 - s) * self.v

    def single_step_forward(self, x: torch.Tensor) -> torch.Tensor:
        self.neuronal_charge(x)
        spike = self.neuronal_fire()
        self.neuronal_reset(spike)
        return spike

    def multi_step_forward(self, x_seq: torch.Tensor) -> torch.Tensor:
        return torch.stack([self.single_step_forward(x) for x in x_seq])


class BaseNode(base.MemoryModule):
    """Common machinery of spiking neurons with one membrane state ``v``."""

    #: subclasses with a kernel form set this to True
    _has_native = False
    #: does single-step mode have a native path as well
    _native_single_step = False

    def __init__(self, v_threshold: float = 1.0, v_reset: Optional[float] = 0.0,
                 surrogate_function: surrogate.SurrogateFunctionBase = surrogate.Sigmoid(),
                 detach_reset: bool = False, step_mode="s", backend="torch", store_v_seq: bool = False):
        assert isinstance(v_reset, float) or v_reset is None
        assert isinstance(v_threshold, float)
        assert isinstance(detach_reset, bool)
        super().__init__()
        self.register_memory("v", 0.0 if v_reset is None else v_reset)
        self.v_threshold = v_threshold
        self.v_reset = v_reset
        self.detach_reset = detach_reset
        self.surrogate_function = surrogate_function
        self.step_mode = step_mode
        self.backend = backend
        self.store_v_seq = store_v_seq
        # read by the Lava exporter; kept as an instance attribute so callers can tune it
        self.lava_s_cale = 1 << 6

    # -- configuration -------------------------------------------------------------
    @property
    def supported_backends(self):
        if not self._has_native:
            return ("torch",)
        if self.step_mode == "s" and not self._native_single_step:
            return ("torch",)
        return _ALL_BACKENDS

    @property
    def store_v_seq(self) -> bool:
        return self._store_v_seq

    @store_v_seq.setter
    def store_v_seq(self, value: bool):
        self._store_v_seq = value
        self.v_seq = None

    def reset(self):
        super().reset()
        self.v_seq = None

    def extra_repr(self):
        return (f"v_threshold={self.v_threshold}, v_reset={self.v_reset}, detach_reset={self.detach_reset}, "
                f"step_mode={self.step_mode}, backend={self.backend}")

    @staticmethod
    def apply_hard_reset(v, spike, v_reset: float):
        return (1.0 - spike) * v + spike * v_reset

    @staticmethod
    def apply_soft_reset(v, spike, v_threshold: float):
        return v - spike * v_threshold

    # -- dynamics hooks ------------------------------------------------------------
    def _eager_step(self, x, v, sg):
        raise NotImplementedError(f"{self._get_name()} must implement _eager_step")

    def _native_sequence(self, x_seq, v, store_v_seq: bool):
        raise NotImplementedError

    def _eager_surrogate(self):
        """In eval mode a spiking surrogate is plain Heaviside (no autograd node)."""
        sg = self.surrogate_function
        if self.training or not getattr(sg, "spiking", True):
            return sg
        return surrogate.heaviside

    def _use_native(self, x: torch.Tensor) -> bool:
        if not (self._has_native and self.native):
            return False
        if not x.is_cuda:
            return False  # CPU tensors always take the eager path
        if not self.training and not getattr(self.surrogate_function, "spiking", True):
            raise NotImplementedError("The native backend only supports spiking surrogate functions. "
                                      "Use backend='torch' for non-spiking surrogate functions.")
        return True

    def _initial_v_value(self) -> float:
        return self.v_reset if self.v_reset is not None else 0.0

    # -- functional protocol -------------------------------------------------------
    def materialize_states(self, inputs, states, step_mode):
        x = inputs[0][0] if step_mode == "m" else inputs[0]
        v = states[0]
        if isinstance(v, float):
            v = torch.full_like(x, v, requires_grad=False)
        elif isinstance(v, torch.Tensor):
            if v.shape != x.shape:
                v = torch.full_like(x, self._initial_v_value(), requires_grad=False)
            elif v.dtype != x.dtype or v.device != x.device:
                v = v.to(dtype=x.dtype, device=x.device)
        return (v, *states[1:])

    def single_step_functional_forward(self, inputs, states, **kwargs):
        x, v = inputs[0], states[0]
        if self._native_single_step and self._use_native(x):
            s, v, _ = self._native_sequence(x.unsqueeze(0), v, False)
            return (s[0],), (v, *states[1:])
        spike, v = self._eager_step(x, v, self._eager_surrogate())
        return (spike,), (v, *states[1:])

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        x_seq, v = inputs[0], states[0]
        if self._use_native(x_seq):
            spike_seq, v, _ = self._native_sequence(x_seq, v, False)
            return (spike_seq,), (v, *states[1:])
        return super().multi_step_functional_forward(inputs, states, **kwargs)

    # -- stateful forward ----------------------------------------------------------
    def _raw_or_materialized_v(self, x_seq):
        """For the native path a float sentinel is passed to the kernel as a scalar: no
        ``full_like`` allocation and no read of an initial-state tensor."""
        v = self._memories["v"]
        if isinstance(v, float):
            return v
        if isinstance(v, torch.Tensor) and v.shape != x_seq.shape[1:]:
            return float(self._initial_v_value())
        return self.materialize_states((x_seq,), (v,), "m")[0]

    def multi_step_forward(self, x_seq: torch.Tensor, *args, **kwargs):
        if len(self._memories) == 1 and not args and self._use_native(x_seq):
            spike_seq, v, v_seq = self._native_sequence(x_seq, self._raw_or_materialized_v(x_seq), self.store_v_seq)
            self._memories["v"] = v
            if self.store_v_seq:
                self.v_seq = v_seq
            return spike_seq
        if not self.store_v_seq:
            return super().multi_step_forward(x_seq, *args, **kwargs)
        inputs = (x_seq, *args)
        states = self.materialize_states(inputs, tuple(self._memories.values()), "m")
        spikes, vs = [], []
        for t in range(x_seq.shape[0]):
            outs, states = self.single_step_functional_forward(tuple(x[t] for x in inputs), states, **kwargs)
            spikes.append(outs)
            vs.append(states[0])
        self._commit(states)
        self.v_seq = torch.stack(vs)
        outs = tuple(torch.stack(o) for o in zip(*spikes))
        return outs[0] if len(outs) == 1 else outs


class NonSpikingBaseNode(nn.Module, base.MultiStepModule):
    """Integrator without spikes; reads out membrane potential over a sequence.
    ``decode``: ``max-mem`` | ``max-abs-mem`` | ``mean-mem`` | ``last_mem`` | None (list)."""

    def __init__(self, decode: Optional[str] = None):
        super().__init__()
        self.decode = decode
        # no ``_step_mode`` is set: like in the reference, ``hasattr(node, "step_mode")`` is False, so ``set_step_mode(net, "s")`` on
        # a network that ends in a non-spiking read-out leaves this node alone (it always consumes a whole sequence)

    @abstractmethod
    def neuronal_charge(self, x: torch.Tensor):
        raise NotImplementedError

    def forward(self, x_seq: torch.Tensor):
        self.v = torch.zeros_like(x_seq[0].detach())
        trace = []
        for t in range(x_seq.shape[0]):
            self.neuronal_charge(x_seq[t])
            trace.append(self.v)
        if self.decode == "max-mem":
            return torch.stack(trace, 0).max(0).values
        if self.decode == "max-abs-mem":
            stack = torch.stack(trace, 0)
            hi, lo = stack.max(0).values, stack.min(0).values
            return torch.where(hi.abs() > lo.abs(), hi, lo)
        if self.decode == "mean-mem":
            return torch.stack(trace, 0).mean(0)
        if self.decode == "last_mem":
            return trace[-1]
        return trace
