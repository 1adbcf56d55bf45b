"""Neurons tied to a training method: membrane-potential batch-norm (MPBN), differentiation on
spike representation (DSR) and online training through time (OTTT / SLTT).

Parity: ``neuron/mpbn.py:13-416``, ``neuron/dsr.py:11-428``, ``neuron/online_learning.py:11-341``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import base, functional, surrogate
from .base_node import BaseNode
from .lif import LIFNode

__all__ = ["MPBNBaseNode", "MPBNLIFNode", "DSRIFNode", "DSRLIFNode", "OTTTLIFNode", "SLTTLIFNode"]


class MPBNBaseNode(BaseNode):
    """Neuron with a BatchNorm (``vbn``) applied to the charged membrane potential.  After
    training, :meth:`re_parameterize_v_threshold` folds the BN into a per-channel threshold so
    that inference needs no normalisation."""

    def __init__(self, v_threshold: float = 1.0, v_reset: Optional[float] = 0.0,
                 surrogate_function=surrogate.Sigmoid(), detach_reset: bool = False, step_mode="s", backend="torch",
                 store_v_seq: bool = False, mpbn: bool = True, out_features=None, out_channels=None,
                 learnable_vth: bool = False, bn_momentum: float = 0.1, bn_decay_momentum: float = 0.94,
                 bn_min_momentum: float = 0.005):
        super().__init__(v_threshold, v_reset, surrogate_function, detach_reset, step_mode, backend, store_v_seq)
        if (out_features is None) == (out_channels is None):
            raise ValueError("Specify exactly one of out_features or out_channels.")
        n = out_channels if out_channels is not None else out_features
        if mpbn:
            self.vbn = nn.BatchNorm2d(n) if out_channels is not None else nn.BatchNorm1d(n)
        else:
            self.vbn = nn.Identity()
        self.register_buffer("mu", None)
        self.register_buffer("sigma2", None)
        self.gamma = self.beta = self.eps = None
        self.fold_bn = self.normalize_residual = self.running_stats = False
        self.bn_momentum, self.bn_decay_momentum, self.bn_min_momentum = bn_momentum, bn_decay_momentum, bn_min_momentum
        self.learnable_vth = learnable_vth
        if learnable_vth:
            self.a = nn.Parameter(torch.zeros(n))      # threshold = exp(a) > 0

    def re_parameterize_v_threshold(self, normalize_residual: bool = False, running_stats: bool = False):
        if isinstance(self.vbn, nn.Identity):
            return
        self.fold_bn = True
        if self.learnable_vth:
            self.v_threshold = torch.exp(self.a.detach())
            del self.a
            self.learnable_vth = False
        self.normalize_residual, self.running_stats = normalize_residual, running_stats
        self.mu, self.sigma2 = self.vbn.running_mean, self.vbn.running_var
        self.gamma, self.beta, self.eps = self.vbn.weight, self.vbn.bias, self.vbn.eps
        self.vbn = nn.Identity()


class MPBNLIFNode(MPBNBaseNode):
    def __init__(self, tau: float = 2.0, decay_input: bool = False, v_threshold: float = 1.0,
                 v_reset: Optional[float] = 0.0, surrogate_function=surrogate.Sigmoid(), detach_reset: bool = False,
                 step_mode="s", backend="torch", store_v_seq: bool = False, mpbn: bool = True, out_features=None,
                 out_channels=None, learnable_vth: bool = False, bn_momentum: float = 0.1,
                 bn_decay_momentum: float = 0.94, bn_min_momentum: float = 0.005):
        assert isinstance(tau, float) and tau > 1.0
        super().__init__(v_threshold, v_reset, surrogate_function, detach_reset, step_mode, backend, store_v_seq, mpbn,
                         out_features, out_channels, learnable_vth, bn_momentum, bn_decay_momentum, bn_min_momentum)
        self.tau, self.decay_input = tau, decay_input

    def _has_bn(self) -> bool:
        return not isinstance(self.vbn, nn.Identity)

    def _normalization_state(self) -> dict:
        """Running statistics as plain values, so the functional forward can stay pure."""
        bn = self.vbn if self._has_bn() else None
        return {
            "running_mean": bn.running_mean.clone() if bn is not None else None,
            "running_var": bn.running_var.clone() if bn is not None else None,
            "num_batches_tracked": bn.num_batches_tracked.clone() if bn is not None else None,
            "mu": self.mu, "sigma2": self.sigma2, "bn_momentum": self.bn_momentum,
        }

    def forward(self, *args, **kwargs):
        stats = self._normalization_state()
        kwargs["_mpbn_stats"] = stats
        out = super().forward(*args, **kwargs)
        if self.training:
            if self._has_bn():
                self.vbn.running_mean.copy_(stats["running_mean"])
                self.vbn.running_var.copy_(stats["running_var"])
                self.vbn.num_batches_tracked.copy_(stats["num_batches_tracked"])
            elif self.fold_bn and not self.learnable_vth:
                self.mu, self.sigma2, self.bn_momentum = stats["mu"], stats["sigma2"], stats["bn_momentum"]
        return out

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        kwargs.setdefault("_mpbn_stats", self._normalization_state())
        return base.MemoryModule.multi_step_functional_forward(self, inputs, states, **kwargs)

    def multi_step_forward(self, x_seq, *args, **kwargs):
        return base.MemoryModule.multi_step_forward(self, x_seq, *args, **kwargs)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        x, v = inputs[0], states[0]
        stats = kwargs.get("_mpbn_stats") or self._normalization_state()
        v = functional.lif_charge(x, v, self.tau, self.decay_input, self.v_reset)
        if self._has_bn():
            factor = 0.0 if self.vbn.momentum is None else self.vbn.momentum
            if self.training:
                stats["num_batches_tracked"].add_(1)
                if self.vbn.momentum is None:
                    factor = 1.0 / float(stats["num_batches_tracked"])
            v = F.batch_norm(v, stats["running_mean"], stats["running_var"], self.vbn.weight, self.vbn.bias,
                             self.training, factor, self.vbn.eps)
        mu, sigma2, mom = stats["mu"], stats["sigma2"], stats["bn_momentum"]
        folded = self.fold_bn and not self.learnable_vth
        if folded and self.training and not (v.ndim == 2 and v.shape[0] == 1):
            dims = 0 if v.ndim == 2 else (0, 2, 3)
            b_mu = v.mean(dim=dims).detach()
            b_var = v.var(dim=dims, unbiased=True).detach()
            if self.running_stats:
                mu = mu.detach() * (1 - mom) + b_mu * mom
                sigma2 = sigma2.detach() * (1 - mom) + b_var * mom
                mom = max(mom * self.bn_decay_momentum, self.bn_min_momentum)
            else:
                mu, sigma2 = b_mu, b_var
            stats["mu"], stats["sigma2"], stats["bn_momentum"] = mu, sigma2, mom
        shape = (1, -1) if v.ndim == 2 else (1, -1, 1, 1)
        if folded:
            th = (self.v_threshold - self.beta) * torch.sqrt(sigma2 + self.eps) / self.gamma + mu
        elif self.learnable_vth:
            th = torch.exp(self.a)
        else:
            th = self.v_threshold
        if self.fold_bn or self.learnable_vth:
            th = th.view(shape)
        diff = v - th
        spike = self.surrogate_function(diff)
        if self.normalize_residual:
            mask = diff <= 0
            sigma = torch.sqrt(sigma2 + self.eps).view(shape)
            normed = (v - mu.view(shape)) / sigma * self.gamma.view(shape) + self.beta.view(shape)
            v = torch.where(mask, normed, v)
        v = functional.voltage_reset(v, spike, self.v_threshold, self.v_reset, self.detach_reset)
        return (spike,), (v, *states[1:])


class _DSRBase(base.MemoryModule):
    """Common part of the DSR neurons: a (possibly trainable) threshold bounded from below."""

    def __init__(self, T, v_threshold, alpha, v_threshold_training, v_threshold_grad_scaling, v_threshold_lower_bound,
                 step_mode, backend):
        assert isinstance(T, int)
        assert isinstance(v_threshold, float) and v_threshold >= v_threshold_lower_bound
        assert isinstance(alpha, float) and 0.0 < alpha <= 1.0
        assert isinstance(v_threshold_lower_bound, float) and v_threshold_lower_bound > 0.0
        assert step_mode == "m"
        super().__init__()
        self.backend = backend
        self.step_mode = step_mode
        self.T = T
        vt = torch.tensor(v_threshold)
        self.v_threshold = nn.Parameter(vt) if v_threshold_training else vt
        self.alpha = alpha
        self.v_threshold_lower_bound = v_threshold_lower_bound
        self.v_threshold_grad_scaling = v_threshold_grad_scaling


class _DSRIFFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, T, v_threshold, alpha, grad_scaling):
        ctx.save_for_backward(inp)
        ctx.T, ctx.v_threshold, ctx.grad_scaling = T, v_threshold, grad_scaling
        mem = torch.zeros_like(inp[0])
        out = []
        for t in range(inp.size(0)):
            mem = mem + inp[t]
            spike = (mem >= alpha * v_threshold).float() * v_threshold
            mem = mem - spike
            out.append(spike)
        return torch.stack(out)

    @staticmethod
    def backward(ctx, grad_output):
        (inp,) = ctx.saved_tensors
        T, vth = ctx.T, ctx.v_threshold
        with torch.no_grad():
            rate = inp.mean(0)
            g = grad_output.mean(0) * T
            gi = torch.where((rate < 0) | (rate > vth), torch.zeros_like(g), g)
            gi = gi.unsqueeze(0).expand(T, *gi.shape) / T
            gv = torch.where(rate <= vth, torch.zeros_like(g), g).sum() * ctx.grad_scaling
        return gi, None, gv, None, None


class DSRIFNode(_DSRBase):
    """IF neuron trained on its rate representation: forward simulates ``T`` steps (spikes of
    height ``v_threshold``, firing at ``alpha * v_threshold``); backward treats the average
    output as ``clamp(mean input, 0, v_threshold)``."""

    DSRIFFunction = _DSRIFFn

    def __init__(self, T: int = 20, v_threshold: float = 6.0, alpha: float = 0.5, v_threshold_training: bool = True,
                 v_threshold_grad_scaling: float = 1.0, v_threshold_lower_bound: float = 0.01, step_mode="m",
                 backend="torch", **kwargs):
        super().__init__(T, v_threshold, alpha, v_threshold_training, v_threshold_grad_scaling,
                         v_threshold_lower_bound, step_mode, backend)

    def extra_repr(self):
        return (f", T={self.T}, init_vth={self.v_threshold}, alpha={self.alpha}, "
                f"vth_bound={self.v_threshold_lower_bound}, vth_g_scale={self.v_threshold_grad_scaling}")

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        vth = self.v_threshold.clamp(min=self.v_threshold_lower_bound)
        return (_DSRIFFn.apply(inputs[0], self.T, vth, self.alpha, self.v_threshold_grad_scaling),), states


class _DSRLIFFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, T, v_threshold, tau, delta_t, alpha, grad_scaling):
        ctx.save_for_backward(inp)
        ctx.T, ctx.v_threshold, ctx.tau, ctx.delta_t, ctx.grad_scaling = T, v_threshold, tau, delta_t, grad_scaling
        mem = torch.zeros_like(inp[0])
        beta = math.exp(-delta_t / tau)
        out = []
        for t in range(inp.size(0)):
            mem = beta * mem + (1 - beta) * inp[t]
            spike = (mem >= alpha * v_threshold).float() * v_threshold
            mem = mem - spike
            out.append(spike / delta_t)
        return torch.stack(out)

    @staticmethod
    def backward(ctx, grad_output):
        (inp,) = ctx.saved_tensors
        T, vth, tau, dt = ctx.T, ctx.v_threshold, ctx.tau, ctx.delta_t
        rate = DSRLIFNode.weight_rate_spikes(inp, tau, dt)
        g = DSRLIFNode.weight_rate_spikes(grad_output, tau, dt) * T
        bound = vth / dt * tau
        inside = (rate > 0) & (rate < bound)
        gi = torch.where(inside, g / tau, torch.zeros_like(g))
        gi = gi.unsqueeze(0).expand(T, *gi.shape) / T
        gv = torch.where(rate <= bound, torch.zeros_like(g), g).sum() * dt * ctx.grad_scaling
        return gi, None, gv, None, None, None, None


class DSRLIFNode(_DSRBase):
    """LIF counterpart of :class:`DSRIFNode` (exponentially weighted rate representation)."""

    DSRLIFFunction = _DSRLIFFn

    def __init__(self, T: int = 20, v_threshold: float = 1.0, tau: float = 2.0, delta_t: float = 0.05,
                 alpha: float = 0.3, v_threshold_training: bool = True, v_threshold_grad_scaling: float = 1.0,
                 v_threshold_lower_bound: float = 0.1, step_mode="m", backend="torch", **kwargs):
        super().__init__(T, v_threshold, alpha, v_threshold_training, v_threshold_grad_scaling,
                         v_threshold_lower_bound, step_mode, backend)
        self.tau, self.delta_t = tau, delta_t

    def extra_repr(self):
        return (f", T={self.T}, init_vth={self.v_threshold}, tau={self.tau}, dt={self.delta_t}, alpha={self.alpha}, "
                f"vth_bound={self.v_threshold_lower_bound}, vth_g_scale={self.v_threshold_grad_scaling}")

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        vth = self.v_threshold.clamp(min=self.v_threshold_lower_bound)
        y = _DSRLIFFn.apply(inputs[0], self.T, vth, self.tau, self.delta_t, self.alpha, self.v_threshold_grad_scaling)
        return (y,), states

    @classmethod
    def weight_rate_spikes(cls, data, tau, delta_t):
        """Exponentially weighted time average over the leading axis."""
        T = data.shape[0]
        w = torch.tensor([math.exp(-1 / tau * (delta_t * T - i * delta_t)) for i in range(1, T + 1)],
                         device=data.device, dtype=data.dtype)
        return torch.tensordot(w, data, dims=([0], [0])) / w.sum()


class _OnlineLIFNode(LIFNode):
    """LIF whose previous potential is detached in training (no gradient through time)."""
    _has_native = False

    def single_step_functional_forward(self, inputs, states, **kwargs):
        v = states[0]
        spike, v = functional.lif_step(inputs[0], v.detach() if self.training else v, self.tau, self.decay_input,
                                       self.v_threshold, self.v_reset,
                                       self.surrogate_function if self.training else surrogate.heaviside,
                                       self.detach_reset)
        return (spike,), (v, *states[1:])


class OTTTLIFNode(_OnlineLIFNode):
    """OTTT neuron: in training it returns ``[spike, trace]`` with the presynaptic trace
    ``a <- a (1 - 1/tau) + s`` (memory ``trace``)."""

    def __init__(self, tau: float = 2.0, decay_input: bool = False, v_threshold: float = 1.0,
                 v_reset: Optional[float] = None, surrogate_function=surrogate.Sigmoid(), detach_reset: bool = True,
                 step_mode="s", backend="torch", store_v_seq: bool = False):
        super().__init__(tau, decay_input, v_threshold, v_reset, surrogate_function, detach_reset, step_mode, backend,
                         store_v_seq)
        assert step_mode == "s", "Please use single-step mode to enable memory-efficient training."
        self.register_memory("trace", None)

    def materialize_states(self, inputs, states, step_mode):
        states = super().materialize_states(inputs, states, step_mode)
        trace = states[1]
        if self.training and trace is None:
            trace = torch.zeros_like(states[0])
        return states[0], trace

    @staticmethod
    def track_trace(spike, trace, tau: float):
        with torch.no_grad():
            return trace * (1.0 - 1.0 / tau) + spike

    def single_step_functional_forward(self, inputs, states, **kwargs):
        (spike,), (v, trace) = super().single_step_functional_forward(inputs, states, **kwargs)
        if not self.training:
            return (spike,), (v, trace)
        trace = self.track_trace(spike, trace, self.tau)
        return (spike, trace), (v, trace)

    def single_step_forward(self, x):
        out = super().single_step_forward(x)
        return list(out) if isinstance(out, tuple) else out


class SLTTLIFNode(_OnlineLIFNode):
    """SLTT neuron: spatial learning through time (temporal gradient paths are cut)."""

    def __init__(self, tau: float = 2.0, decay_input: bool = True, v_threshold: float = 1.0,
                 v_reset: Optional[float] = 0.0, surrogate_function=surrogate.Sigmoid(), detach_reset: bool = True,
                 step_mode="s", backend="torch", store_v_seq: bool = False):
        super().__init__(tau, decay_input, v_threshold, v_reset, surrogate_function, detach_reset, step_mode, backend,
                         store_v_seq)
        assert step_mode == "s", "Please use single-step mode to enable memory-efficient training."
