"""Tempotron: a timing-based neuron whose membrane potential is the weighted sum of double-exponential
post-synaptic potentials started at the input spike times (``spikingjelly/timing_based/neuron.py:10-192``)."""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["Tempotron"]


class Tempotron(nn.Module):
    """Input: ``[batch, in_features]`` spike times (negative = no spike).  ``forward(x, ret_type)`` returns the
    voltage trace ``[batch, out_features, T]`` (``"v"``), its maximum over time (``"v_max"``) or output spike times
    (``"spikes"``: arg-max time with a soft-arg-max gradient, negated for neurons that stay below threshold).
    The weight lives at ``model.summation_layer.weight`` for checkpoint compatibility."""

    def __init__(self, in_features: int, out_features: int, T: int, tau: float = 15.0, tau_s: float = 15.0 / 4,
                 v_threshold: float = 1.0) -> None:
        super().__init__()
        if in_features <= 0 or out_features <= 0 or T <= 0:
            raise ValueError("in_features, out_features, and T must be positive.")
        if tau <= 0 or tau_s <= 0 or v_threshold <= 0 or tau == tau_s:
            raise ValueError("tau and tau_s must be positive and different; v_threshold must be positive.")
        self.in_features, self.out_features, self.T = in_features, out_features, T
        self.tau, self.tau_s, self.v_threshold = tau, tau_s, v_threshold
        self._make_layer(in_features, out_features)
        # normalise the kernel so that a single input of weight 1 peaks exactly at the threshold
        t_peak = tau * tau_s * math.log(tau / tau_s) / (tau - tau_s)
        self.v0 = v_threshold / (math.exp(-t_peak / tau) - math.exp(-t_peak / tau_s))

    def _make_layer(self, in_features: int, out_features: int) -> None:
        self.model = nn.Module()
        self.model.summation_layer = nn.Linear(in_features, out_features, bias=False)

    def _summation(self) -> nn.Linear:
        return self.model.summation_layer

    @staticmethod
    def _psp_kernel(t: torch.Tensor, tau: float, tau_s: float) -> torch.Tensor:
        t = t.clamp_min(0)            # zero before the spike: exp(0) - exp(0)
        return torch.exp(-t / tau) - torch.exp(-t / tau_s)

    def mse_loss(self, v_max: torch.Tensor, label: torch.Tensor) -> torch.Tensor:
        """Squared distance to the threshold of every neuron whose firing decision is wrong, averaged over the batch."""
        fired = (v_max >= self.v_threshold).to(v_max.dtype)
        wrong = (fired != F.one_hot(label, self.out_features)).to(v_max.dtype)
        return ((v_max - self.v_threshold) * wrong).square().sum() / label.shape[0]

    def forward(self, in_spikes: torch.Tensor, ret_type: str) -> torch.Tensor:
        steps = torch.arange(self.T, device=in_spikes.device).view(1, 1, self.T)
        t_spike = in_spikes.unsqueeze(-1)
        psp = self.v0 * self._psp_kernel(steps - t_spike, self.tau, self.tau_s) * (t_spike >= 0).float()
        voltage = self._summation()(psp.transpose(1, 2)).transpose(1, 2)
        if ret_type == "v":
            return voltage
        peak, hard = voltage.max(dim=2)
        if ret_type == "v_max":
            return peak
        if ret_type == "spikes":
            soft = (F.softmax(voltage * self.T, dim=2) * steps).sum(dim=2)
            sign = (peak >= self.v_threshold).to(voltage.dtype) * 2 - 1
            hard, soft = hard * sign, soft * sign
            return soft + (hard - soft).detach()
        raise ValueError(f"Invalid out_voltage_type: {ret_type}. Must be 'v', 'v_max', or 'spikes'")
