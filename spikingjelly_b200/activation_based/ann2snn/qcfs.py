"""Signed QCFS sequence encoder: turn an analog activation into ``T`` steps of signed spikes whose sum
is the activation quantised to ``scale * round(x / scale)`` (clipped to ``+-T * scale``).  Two
``ActivationAwareIFNode`` populations (positive / negative part, initial potential = half a threshold)
integrate ``|x| / T`` per step; elements whose emitted count misses the target by a rounding-boundary
effect are re-encoded as a burst of exactly the target count.
Parity: ``spikingjelly/activation_based/ann2snn/qcfs.py:12-458``."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import neuron, quantize, surrogate

__all__ = ["SignedQCFSSequenceEncoder"]


class SignedQCFSSequenceEncoder(nn.Module):
    def __init__(self, scale: torch.Tensor, time_steps: int, *, neuron_backend: str = "torch", channel_dim: int = -1,
                 collect_statistics: bool = True, name: str = "activation") -> None:
        super().__init__()
        if not isinstance(scale, torch.Tensor):
            raise TypeError("scale must be a torch.Tensor.")
        if scale.dim() != 1 or not torch.isfinite(scale).all() or not (scale > 0).all():
            raise ValueError("scale must be a finite positive one-dimensional tensor.")
        if not isinstance(time_steps, int) or isinstance(time_steps, bool):
            raise TypeError("time_steps must be an integer.")
        if time_steps <= 0:
            raise ValueError("time_steps must be positive.")
        if not isinstance(channel_dim, int) or isinstance(channel_dim, bool):
            raise TypeError("channel_dim must be an integer.")
        if neuron_backend not in ("torch", "triton", "cuda"):
            raise ValueError(f"Unsupported ActivationAwareIFNode backend={neuron_backend!r}.")
        self.name, self.time_steps, self.channel_dim = str(name), time_steps, channel_dim
        self.collect_statistics = bool(collect_statistics)
        kw = dict(v_threshold=scale, v_offset=0.5 * scale, channel_dim=channel_dim, v_reset=None,
                  surrogate_function=surrogate.DeterministicPass(), step_mode="m", backend="torch")
        self.positive_neuron = neuron.ActivationAwareIFNode(**kw)
        self.negative_neuron = neuron.ActivationAwareIFNode(**kw)
        self.metric_scope = "activation"
        self._clear_statistics()

    def _clear_statistics(self) -> None:
        self.positive_spike_rate = self.negative_spike_rate = 0.0
        self.positive_spike_count = self.negative_spike_count = self.spike_value_count = 0
        self.local_relative_l2 = self.boundary_correction_fraction = 0.0

    def _channel_scale(self, value: torch.Tensor) -> torch.Tensor:
        s = self.positive_neuron.v_threshold.to(value)
        shape = [1] * value.dim()
        shape[self.channel_dim % value.dim()] = s.numel()
        return s.reshape(shape)

    def _encode_nonnegative(self, node, value: torch.Tensor):
        T = self.time_steps
        scale = self._channel_scale(value)
        node.reset()
        spikes = node(value.unsqueeze(0).expand(T, *value.shape) / T)
        desired = torch.round(value / scale).clamp(0, T)
        mismatch = spikes.sum(0).ne(desired)
        if mismatch.any():
            t = torch.arange(T, device=value.device).reshape(T, *([1] * value.dim()))
            burst = (t < desired.unsqueeze(0)).to(spikes.dtype)
            spikes = torch.where(mismatch.unsqueeze(0), burst, spikes)
            if self.collect_statistics and not torch.equal(spikes.sum(0), desired):
                raise RuntimeError("Signed QCFS encoding failed to replay target counts.")
        return spikes, mismatch

    def encode(self, value: torch.Tensor, metric_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``value [...]`` -> signed spike sequence ``[T, ...]`` scaled by the channel scale."""
        if not torch.is_floating_point(value):
            raise ValueError("Signed QCFS encoding requires a floating-point tensor.")
        if value.dim() == 0:
            raise ValueError("Signed QCFS encoding requires at least one dimension.")
        cd = self.channel_dim % value.dim()
        if value.shape[cd] != self.positive_neuron.v_threshold.numel():
            raise ValueError("Input channel size does not match the QCFS scale.")
        pos, pos_fix = self._encode_nonnegative(self.positive_neuron, F.relu(value))
        neg, neg_fix = self._encode_nonnegative(self.negative_neuron, F.relu(-value))
        seq = (pos - neg) * self._channel_scale(value)
        if self.collect_statistics:
            p, n, rec, ref, count = pos.detach(), neg.detach(), seq.sum(0), value, value.numel()
            if metric_mask is not None:
                mask = metric_mask.to(device=value.device, dtype=torch.bool)
                expect = value.shape[:cd] + value.shape[cd + 1:]
                if mask.shape != expect:
                    raise ValueError(f"metric_mask shape must match value dimensions excluding channel_dim: expected {tuple(expect)}, "
                                     f"got {tuple(mask.shape)}.")
                if not mask.any():
                    raise ValueError("metric_mask must select at least one element.")
                full = mask.unsqueeze(cd).expand(value.shape)
                p, n, pos_fix, neg_fix, rec, ref, count = p[:, full], n[:, full], pos_fix[full], neg_fix[full], rec[full], ref[full], int(full.count_nonzero())
            self.positive_spike_rate, self.negative_spike_rate = float(p.mean()), float(n.mean())
            self.positive_spike_count, self.negative_spike_count = int(p.count_nonzero()), int(n.count_nonzero())
            self.spike_value_count = int(p.numel())
            self.boundary_correction_fraction = (int(pos_fix.count_nonzero()) + int(neg_fix.count_nonzero())) / (2 * count)
            self.local_relative_l2 = float(torch.linalg.vector_norm((rec - ref).float()) / torch.linalg.vector_norm(ref.float()).clamp_min(1e-12))
            if not math.isfinite(self.local_relative_l2):
                raise ValueError("Signed QCFS local relative L2 must be finite.")
        return seq

    def reconstruct(self, value: torch.Tensor) -> torch.Tensor:
        """The value the encoded sequence sums to (differentiable through the straight-through quantiser)."""
        if not torch.is_floating_point(value):
            raise ValueError("Signed QCFS reconstruction requires floating point.")
        if value.dim() == 0:
            raise ValueError("Signed QCFS reconstruction requires at least one dimension.")
        if value.shape[self.channel_dim % value.dim()] != self.positive_neuron.v_threshold.numel():
            raise ValueError("Input channel size does not match the QCFS scale.")
        scale = self._channel_scale(value)
        pos = quantize.multi_level_spike_count(F.relu(value) / scale, self.time_steps)
        neg = quantize.multi_level_spike_count(F.relu(-value) / scale, self.time_steps)
        return (pos - neg) * scale

    def forward(self, value_seq: torch.Tensor, metric_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Re-encode a sequence: its sum over time is encoded afresh."""
        if value_seq.dim() < 2 or value_seq.shape[0] <= 0:
            raise ValueError("value_seq must have a non-empty leading time dimension.")
        return self.encode(value_seq.sum(0), metric_mask)

    def statistics(self) -> Dict[str, object]:
        peaks = [float(n.v.detach().abs().max()) if isinstance(n.v, torch.Tensor) else abs(float(n.v))
                 for n in (self.positive_neuron, self.negative_neuron)]
        return {"name": self.name, "backend": self.positive_neuron.backend, "positive_spike_rate": self.positive_spike_rate,
                "negative_spike_rate": self.negative_spike_rate, "positive_spike_count": self.positive_spike_count,
                "negative_spike_count": self.negative_spike_count, "spike_value_count": self.spike_value_count,
                "local_relative_l2": self.local_relative_l2, "metric_scope": self.metric_scope,
                "boundary_correction_fraction": self.boundary_correction_fraction, "membrane_abs_max": max(peaks)}
