"""Attention modules for spiking networks.

``SpikingSelfAttention`` is softmax-free: with spike matrices Q, K, V per head,
``out = (V K^T) Q * 0.125`` in channel-major layout ``[Cph, L]`` — equivalently
``Q (K^T V)`` token-major — followed by a LIF with threshold 0.5.  On CUDA with the
native backend the two products and the scaling run in the fused SSA kernel.

Parity: ``spikingjelly/activation_based/layer/attention.py`` — TemporalWiseAttention
:61-148, MultiDimensionalAttention :151-242, SpikingSelfAttention :245-387,
QKAttention family :390-602.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import base, neuron
from .container import SeqToANNContainer

__all__ = ["TemporalWiseAttention", "MultiDimensionalAttention", "SpikingSelfAttention", "QKAttention",
           "TokenQKAttention", "ChannelQKAttention"]


class _SqueezeExcite3d(nn.Module):
    """sigmoid(MLP(avgpool) + MLP(maxpool)) along dim 1 (optionally after swapping dims 1, 2)."""

    def __init__(self, planes, ratio, channel_axis=False):
        super().__init__()
        self.channel_axis = channel_axis
        self.avg_pool, self.max_pool = nn.AdaptiveAvgPool3d(1), nn.AdaptiveMaxPool3d(1)
        self.sharedMLP = nn.Sequential(nn.Conv3d(planes, planes // ratio, 1, bias=False), nn.ReLU(),
                                       nn.Conv3d(planes // ratio, planes, 1, bias=False))

    def forward(self, x):
        if self.channel_axis:
            x = x.transpose(1, 2)
        score = torch.sigmoid(self.sharedMLP(self.avg_pool(x)) + self.sharedMLP(self.max_pool(x)))
        return score.transpose(1, 2) if self.channel_axis else score


class _SpatialGate(nn.Module):
    def __init__(self, kernel_size):
        super().__init__()
        self.conv = nn.Conv2d(2, 1, kernel_size, padding=3 if kernel_size == 7 else 1, bias=False)

    def forward(self, x):
        x = x.flatten(1, 2)
        pooled = torch.cat((x.mean(dim=1, keepdim=True), x.max(dim=1, keepdim=True).values), dim=1)
        return torch.sigmoid(self.conv(pooled)).unsqueeze(1)


class TemporalWiseAttention(nn.Module, base.MultiStepModule):
    """Squeeze-and-excitation over the time axis: each step of ``[T, N, *]`` is rescaled."""

    def __init__(self, T: int, reduction: int = 16, dimension: int = 4):
        super().__init__()
        self._step_mode = "m"
        assert dimension in (2, 4), "dimension must be 4 or 2"
        if dimension == 2:
            self.avg_pool, self.max_pool = nn.AdaptiveAvgPool1d(1), nn.AdaptiveMaxPool1d(1)
        else:
            self.avg_pool, self.max_pool = nn.AdaptiveAvgPool3d(1), nn.AdaptiveMaxPool3d(1)
        assert T >= reduction, "reduction cannot be greater than T"
        self.sharedMLP = nn.Sequential(nn.Linear(T, T // reduction, bias=False), nn.ReLU(),
                                       nn.Linear(T // reduction, T, bias=False))

    def forward(self, x_seq: torch.Tensor):
        assert x_seq.dim() in (3, 5), ValueError(
            f"expected 3D or 5D input with shape [T, N, M] or [T, N, C, H, W], but got input with shape {x_seq.shape}")
        x = x_seq.transpose(0, 1)
        n, t = x.shape[:2]
        score = torch.sigmoid(self.sharedMLP(self.avg_pool(x).view(n, t)) + self.sharedMLP(self.max_pool(x).view(n, t)))
        return (x * score.view(n, t, *((1,) * (x.ndim - 2)))).transpose(0, 1)


class MultiDimensionalAttention(nn.Module, base.MultiStepModule):
    """Temporal, channel and spatial attention applied in sequence to ``[T, N, C, H, W]``."""

    def __init__(self, T: int, C: int, reduction_t: int = 16, reduction_c: int = 16, kernel_size=3):
        super().__init__()
        self._step_mode = "m"
        assert T >= reduction_t, "reduction_t cannot be greater than T"
        assert C >= reduction_c, "reduction_c cannot be greater than C"
        assert kernel_size in (3, 7), "kernel size must be 3 or 7"
        self.ta = _SqueezeExcite3d(T, reduction_t)
        self.ca = _SqueezeExcite3d(C, reduction_c, channel_axis=True)
        self.sa = _SpatialGate(kernel_size)
        self.relu = nn.ReLU()

    def forward(self, x: torch.Tensor):
        assert x.dim() == 5, ValueError(
            f"expected 5D input with shape [T, N, C, H, W], but got input with shape {x.shape}")
        x = x.transpose(0, 1)
        out = self.ta(x) * x
        out = self.ca(out) * out
        out = self.sa(out) * out
        return self.relu(out).transpose(0, 1)


def _lif(backend, v_threshold=1.0):
    return neuron.LIFNode(tau=2.0, v_threshold=v_threshold, detach_reset=True, step_mode="m", backend=backend)


class _BackendFanout:
    """Mixin: ``backend`` reads/sets the backend of the LIF children named in ``_lifs``."""
    _lifs = ()

    @property
    def backend(self):
        return getattr(self, self._lifs[0]).backend

    @backend.setter
    def backend(self, value: str):
        for n in self._lifs:
            getattr(self, n).backend = value


class SpikingSelfAttention(_BackendFanout, nn.Module, base.MultiStepModule):
    """Spikformer self-attention on ``[T, N, C, L]``."""
    _lifs = ("qkv_lif", "attn_lif", "proj_lif")

    def __init__(self, dim, num_heads=8, backend: str = "torch"):
        super().__init__()
        if dim % num_heads != 0:
            raise ValueError(f"dim {dim} should be divided by num_heads {num_heads}.")
        self._step_mode = "m"
        self.dim, self.num_heads, self.head_dim, self.scale = dim, num_heads, dim // num_heads, 0.125
        self.qkv_conv_bn = SeqToANNContainer(nn.Conv1d(dim, dim * 3, kernel_size=1, stride=1, bias=False),
                                             nn.BatchNorm1d(dim * 3))
        self.qkv_lif = _lif(backend)
        self.attn_lif = _lif(backend, 0.5)
        self.proj_conv_bn = SeqToANNContainer(nn.Conv1d(dim, dim, kernel_size=1, stride=1, bias=False),
                                              nn.BatchNorm1d(dim))
        self.proj_lif = _lif(backend)

    @staticmethod
    def _ssa_kernel_torch(qkv, scale):
        """``qkv``: ``[T, N, 3, heads, Cph, L]`` -> ``[T, N, heads, Cph, L]``."""
        q, k, v = qkv.unbind(2)
        return ((v @ k.transpose(-2, -1)) @ q) * scale

    def forward(self, x_seq: torch.Tensor):
        if x_seq.ndim != 4:
            raise ValueError(f"expected 4D input with shape [T, N, C, L], but got input with shape {x_seq.shape}")
        T, N, C, L = x_seq.shape
        qkv = self.qkv_lif(self.qkv_conv_bn(x_seq))
        local = qkv.shape[2] // 3
        if local % self.num_heads != 0:
            raise ValueError(f"local qkv dim {local} is not divisible by num_heads={self.num_heads}.")
        qkv = qkv.reshape(T, N, 3, self.num_heads, local // self.num_heads, L)
        attn = self._ssa_kernel_torch(qkv, self.scale)
        attn = self.attn_lif(attn).reshape(T, N, local, L)
        return self.proj_lif(self.proj_conv_bn(attn))

    def extra_repr(self):
        return f"dim={self.dim}, num_heads={self.num_heads}, backend={self.backend}"


class QKAttention(_BackendFanout, nn.Module, base.MultiStepModule):
    """QKFormer attention: a spike mask computed from Q (summed over tokens or channels,
    then LIF with threshold 0.5) gates K."""
    _lifs = ("qk_lif", "attn_lif", "proj_lif")

    def __init__(self, dim: int, num_heads: int = 8, qka_type: str = "token", backend: str = "torch"):
        super().__init__()
        if dim % num_heads != 0:
            raise ValueError(f"dim {dim} should be divided by num_heads {num_heads}.")
        if qka_type not in ("token", "channel"):
            raise ValueError(f"qka_type should be either 'token' or 'channel', but got {qka_type}.")
        self._step_mode = "m"
        self.dim, self.num_heads, self.head_dim, self._qka_type = dim, num_heads, dim // num_heads, qka_type
        self.qk_conv_bn = SeqToANNContainer(nn.Conv1d(dim, dim * 2, kernel_size=1, stride=1, bias=False),
                                            nn.BatchNorm1d(dim * 2))
        self.qk_lif = _lif(backend)
        self.sum_dim = 3 if qka_type == "token" else 4
        self.attn_lif = _lif(backend, 0.5)
        self.proj_conv_bn = SeqToANNContainer(nn.Conv1d(dim, dim, kernel_size=1, stride=1, bias=False),
                                              nn.BatchNorm1d(dim))
        self.proj_lif = _lif(backend)

    @property
    def qka_type(self):
        return self._qka_type

    def forward(self, x_seq):
        if x_seq.ndim != 4:
            raise ValueError(f"expected 4D input with shape [T, N, C, L], but got input with shape {x_seq.shape}")
        T, N, C, L = x_seq.shape
        qk = self.qk_lif(self.qk_conv_bn(x_seq)).reshape(T, N, 2, self.num_heads, C // self.num_heads, L)
        q, k = qk.unbind(2)
        gate = self.attn_lif(q.sum(dim=self.sum_dim, keepdim=True))
        out = (gate * k).flatten(2, 3)
        return self.proj_lif(self.proj_conv_bn(out))

    def extra_repr(self):
        return f"dim={self.dim}, num_heads={self.num_heads}, qka_type={self.qka_type}, backend={self.backend}"


class TokenQKAttention(QKAttention):
    def __init__(self, dim: int, num_heads: int = 8, backend: str = "torch"):
        super().__init__(dim, num_heads, qka_type="token", backend=backend)


class ChannelQKAttention(QKAttention):
    def __init__(self, dim: int, num_heads: int = 8, backend: str = "torch"):
        super().__init__(dim, num_heads, qka_type="channel", backend=backend)
