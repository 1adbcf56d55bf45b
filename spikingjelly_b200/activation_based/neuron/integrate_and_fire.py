"""Integrate-and-fire family.

Parity: ``neuron/integrate_and_fire.py`` — ``SimpleIFNode`` :28-117, ``IFNode``
:120-369, ``HalfThresholdIFNode`` :372-533, ``ActivationAwareIFNode`` :536-1149,
``NonSpikingIFNode`` :1152-1182.
"""
from __future__ import annotations

import numbers
from typing import Optional, Tuple, Union

import torch

from .. import base, functional, surrogate
from .base_node import BaseNode, NonSpikingBaseNode, SimpleBaseNode

__all__ = ["SimpleIFNode", "IFNode", "HalfThresholdIFNode", "ActivationAwareIFNode", "NonSpikingIFNode"]


class SimpleIFNode(SimpleBaseNode):
    def neuronal_charge(self, x):
        self.v = self.v + x


class IFNode(BaseNode):
    """``h = v + x``."""
    _has_native = True
    _native_single_step = True

    def _eager_step(self, x, v, sg):
        return functional.if_step(x, v, self.v_threshold, self.v_reset, sg, self.detach_reset)

    def _native_sequence(self, x_seq, v, store_v_seq):
        return functional.if_multi_step_cuda(x_seq, v, self.v_threshold, self.v_reset, self.surrogate_function,
                                             self.detach_reset, store_v_seq)


class HalfThresholdIFNode(BaseNode):
    """Soft-reset IF whose potential starts (and resets) at ``v_threshold / 2`` — the
    initialisation that minimises the ANN-to-SNN conversion error."""

    def __init__(self, v_threshold: float = 1.0, surrogate_function=surrogate.Sigmoid(), detach_reset=False,
                 step_mode="s", backend="torch", store_v_seq=False):
        if isinstance(v_threshold, torch.Tensor):
            if v_threshold.numel() != 1:
                raise ValueError("v_threshold must be scalar finite positive.")
            v_threshold = float(v_threshold)
        elif not isinstance(v_threshold, numbers.Real):
            raise TypeError("v_threshold must be a real number.")
        v_threshold = float(v_threshold)
        if not (v_threshold > 0.0 and v_threshold < float("inf")):
            raise ValueError("v_threshold must be finite positive.")
        super().__init__(v_threshold, None, surrogate_function, detach_reset, step_mode, backend, store_v_seq)
        self.set_reset_value("v", self.v_threshold / 2.0)
        self.v = self.v_threshold / 2.0

    def _initial_v_value(self):
        return self.v_threshold / 2.0

    def _eager_surrogate(self):
        return self.surrogate_function

    def _eager_step(self, x, v, sg):
        return functional.if_step(x, v, self.v_threshold, None, sg, self.detach_reset)


class ActivationAwareIFNode(base.MemoryModule):
    """IF neuron with per-channel threshold and offset buffers: fires on
    ``h + v_offset - v_threshold >= 0``.  ``channel_dim`` indexes the single-step input."""

    def __init__(self, v_threshold: Union[float, torch.Tensor] = 1.0, v_offset: Union[float, torch.Tensor] = 0.0,
                 channel_dim: int = -1, v_reset: Optional[float] = None, surrogate_function=surrogate.Sigmoid(),
                 detach_reset: bool = False, step_mode: str = "s", backend: str = "torch", store_v_seq: bool = False):
        super().__init__()
        if base.canonical_backend(backend) not in ("torch", "cuda"):
            raise ValueError(f"Unsupported backend={backend!r}.")
        if base.canonical_backend(backend) == "cuda" and step_mode != "m":
            raise ValueError("ActivationAwareIFNode native backend requires step_mode='m'.")
        if v_reset is not None and not isinstance(v_reset, float):
            raise ValueError(f"v_reset must be a float or None, got {type(v_reset).__name__}.")
        for name, val, typ in (("detach_reset", detach_reset, bool), ("store_v_seq", store_v_seq, bool),
                               ("channel_dim", channel_dim, int)):
            if not isinstance(val, typ):
                raise ValueError(f"{name} must be {typ.__name__}.")
        th, off = torch.as_tensor(v_threshold), torch.as_tensor(v_offset)
        self._check_threshold(th)
        self._check_offset(off)
        self.register_buffer("v_threshold", th.clone().detach())
        self.register_buffer("v_offset", off.clone().detach())
        self.channel_dim = channel_dim
        self.v_reset = v_reset
        self.detach_reset = detach_reset
        self.surrogate_function = surrogate_function
        self.register_memory("v", 0.0 if v_reset is None else v_reset)
        self.store_v_seq = store_v_seq
        self.step_mode = step_mode
        self.backend = backend

    @staticmethod
    def _check_threshold(t: torch.Tensor) -> None:
        if t.dim() > 1:
            raise ValueError(f"v_threshold must be a scalar or 1D tensor, but got shape {tuple(t.shape)}.")
        t = t if torch.is_floating_point(t) else t.to(torch.float)
        if not torch.isfinite(t).all() or not (t > 0).all():
            raise ValueError("v_threshold must contain finite positive values.")

    @staticmethod
    def _check_offset(t: torch.Tensor) -> None:
        if t.dim() > 1:
            raise ValueError(f"v_offset must be a scalar or 1D tensor, but got shape {tuple(t.shape)}.")
        t = t if torch.is_floating_point(t) else t.to(torch.float)
        if not torch.isfinite(t).all():
            raise ValueError("v_offset must contain finite values.")

    @property
    def supported_backends(self) -> Tuple[str, ...]:
        return ("torch",) if self.step_mode == "s" else ("torch", "cuda", "triton")

    @property
    def store_v_seq(self) -> bool:
        return self._store_v_seq

    @store_v_seq.setter
    def store_v_seq(self, value: bool) -> None:
        self._store_v_seq = value
        self.v_seq = None

    def reset(self):
        super().reset()
        self.v_seq = None

    def _canonical_channel_dim(self, x: torch.Tensor) -> int:
        d = self.channel_dim + (x.dim() if self.channel_dim < 0 else 0)
        if d < 0 or d >= x.dim():
            raise ValueError(f"channel_dim={self.channel_dim} is out of range for input with {x.dim()} dimensions.")
        return d

    def _broadcast_parameter(self, param, x, name):
        param = param.to(device=x.device, dtype=x.dtype)
        if param.dim() == 0:
            return param
        d = self._canonical_channel_dim(x)
        if param.numel() != x.shape[d]:
            raise ValueError(f"{name} has length {param.numel()}, but input shape {tuple(x.shape)} has "
                             f"{x.shape[d]} channels at channel_dim={self.channel_dim}.")
        shape = [1] * x.dim()
        shape[d] = param.numel()
        return param.view(shape)

    def materialize_states(self, inputs, states, step_mode):
        x = inputs[0][0] if step_mode == "m" else inputs[0]
        v = states[0]
        if isinstance(v, float):
            v = torch.full_like(x, v, requires_grad=False)
        elif isinstance(v, torch.Tensor):
            if v.shape != x.shape:
                v = torch.full_like(x, self.v_reset if self.v_reset is not None else 0.0, requires_grad=False)
            elif v.dtype != x.dtype or v.device != x.device:
                v = v.to(dtype=x.dtype, device=x.device)
        return (v, *states[1:])

    def _step(self, x, v, sg):
        th = self._broadcast_parameter(self.v_threshold, x, "v_threshold")
        off = self._broadcast_parameter(self.v_offset, x, "v_offset")
        return functional.activation_aware_if_step(x, v, th, off, self.v_reset, sg, self.detach_reset)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        if self.native:
            raise RuntimeError("ActivationAwareIFNode single-step forward supports only backend='torch'; "
                               "refusing implicit backend fallback.")
        spike, v = self._step(inputs[0], states[0], self.surrogate_function)
        return (spike,), (v, *states[1:])

    def _inference_sequence(self, x_seq, v, store_v_seq):
        if self.training:
            raise RuntimeError("ActivationAwareIFNode native backend supports inference only; call eval() first.")
        if not getattr(self.surrogate_function, "spiking", True):
            raise RuntimeError("ActivationAwareIFNode native backend requires a spiking surrogate function.")
        if torch.is_grad_enabled() and any(isinstance(t, torch.Tensor) and t.requires_grad
                                           for t in (x_seq, v, self.v_threshold, self.v_offset)):
            raise RuntimeError("ActivationAwareIFNode native backend does not support autograd.")
        th = self._broadcast_parameter(self.v_threshold, x_seq[0], "v_threshold")
        off = self._broadcast_parameter(self.v_offset, x_seq[0], "v_offset")
        return functional.activation_aware_if_sequence(x_seq, v, th, off, self.v_reset, store_v_seq)

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        if self.native:
            s, v, _ = self._inference_sequence(inputs[0], states[0], False)
            return (s,), (v,)
        outs, v = [], states[0]
        for t in range(inputs[0].shape[0]):
            s, v = self._step(inputs[0][t], v, self.surrogate_function)
            outs.append(s)
        return (torch.stack(outs),), (v, *states[1:])

    def multi_step_forward(self, x_seq, *args, **kwargs):
        if not self.store_v_seq:
            return super().multi_step_forward(x_seq, *args, **kwargs)
        states = self.materialize_states((x_seq, *args), tuple(self._memories.values()), "m")
        if self.native:
            spike_seq, v, v_seq = self._inference_sequence(x_seq, states[0], True)
        else:
            spikes, vs, v = [], [], states[0]
            for t in range(x_seq.shape[0]):
                s, v = self._step(x_seq[t], v, self.surrogate_function)
                spikes.append(s)
                vs.append(v)
            spike_seq, v_seq = torch.stack(spikes), torch.stack(vs)
        self.v = v
        self.v_seq = v_seq
        return spike_seq

    def extra_repr(self):
        return (f"v_threshold_shape={tuple(self.v_threshold.shape)}, v_offset_shape={tuple(self.v_offset.shape)}, "
                f"channel_dim={self.channel_dim}, v_reset={self.v_reset}, detach_reset={self.detach_reset}, "
                f"step_mode={self.step_mode}, backend={self.backend}")


class NonSpikingIFNode(NonSpikingBaseNode):
    def neuronal_charge(self, x):
        self.v = self.v + x
