"""Fused execution of the ``Conv2d -> BatchNorm2d -> LIF / IF`` triple that the plain (VGG-style) spiking networks are made of.

On a CUDA device with 16-bit compute (a 16-bit input or CUDA autocast) the triple runs as a channels-last cuDNN convolution
whose output ``[T*N, H, W, C]`` goes as rows ``[T, N*H*W, C]`` into the fused BatchNorm + neuron kernels
(``ops/csrc/bn_lif.cu``): no NCHW <-> NHWC conversion, no stand-alone BatchNorm kernels, nothing saved for backward but the
convolution output.  The result is returned as a ``[T, N, C, H, W]`` view of channels-last memory, which pooling layers and
the next convolution consume as it is.  :func:`conv_bn_lif` is used by ``VGGBlock`` of the CIFAR10-DVS example network and,
through :func:`run_sequential`, by ``SpikingVGG.features``; everything else falls back to the modules' own forward.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..activation_based import base
from ..ops.bn_lif import bn_lif
from ..ops import conv as conv_ops
from ._resnet_fused import _compute_dtype, _init_v, _spec, bn_is_fusable

__all__ = ["eligible", "conv_bn_lif", "run_sequential"]


def eligible(conv, bn, sn, x_seq: torch.Tensor) -> bool:
    if not (torch.is_tensor(x_seq) and x_seq.is_cuda and x_seq.ndim == 5) or _compute_dtype(x_seq) is None:
        return False
    if not isinstance(conv, nn.Conv2d):
        return False
    if conv.padding_mode != "zeros" or isinstance(conv.padding, str):
        return False
    if not bn_is_fusable(bn):
        return False
    if getattr(sn, "step_mode", "s") != "m" or not getattr(sn, "native", False) or _spec(sn) is None:
        return False
    if getattr(sn, "store_v_seq", False):
        return False
    # only from the reset state: the fused kernels start every sequence at the initial potential
    v = sn._memories.get("v") if hasattr(sn, "_memories") else None
    return isinstance(v, float) and v == (sn.v_reset if sn.v_reset is not None else 0.0)


def conv_bn_lif(conv, bn, sn, x_seq: torch.Tensor) -> torch.Tensor:
    """``x_seq``: ``[T, N, C, H, W]`` -> spikes ``[T, N, C', H', W']`` (a view of channels-last memory)."""
    T, N = x_seq.shape[:2]
    dt = _compute_dtype(x_seq)
    h = x_seq.flatten(0, 1).to(dt).contiguous(memory_format=torch.channels_last)
    with torch.autocast("cuda", enabled=False):
        if conv_ops.supports(conv, h):
            # implicit GEMM on the tensor cores.  Without a bias the epilogue's column sums serve the batch norm;
            # with one the sums are taken again after the add (a batch norm in training mode cancels the bias anyway)
            training = bn.training or bn.running_mean is None
            rows, stats, (H, W) = conv_ops.conv2d_rows(h.permute(0, 2, 3, 1), conv.weight, conv.stride, conv.padding, conv.dilation,
                                                       want_stats=training and conv.bias is None)
            if conv.bias is not None:
                rows = rows + conv.bias.to(dt)
            C = rows.shape[1]
            out = bn_lif(rows.view(T, N * H * W, C), bn, _spec(sn), v_init=_init_v(sn), stats=stats)
        else:
            w = conv.weight.to(dtype=dt, memory_format=torch.channels_last)
            b = None if conv.bias is None else conv.bias.to(dt)
            y = F.conv2d(h, w, b, conv.stride, conv.padding, conv.dilation, conv.groups)
            TN, C, H, W = y.shape
            rows = y.permute(0, 2, 3, 1)
            if not rows.is_contiguous():
                rows = rows.contiguous()
            out = bn_lif(rows.reshape(T, N * H * W, C), bn, _spec(sn), v_init=_init_v(sn))
    base.elide_states([sn])
    return out.view(T, N, H, W, C).permute(0, 1, 4, 2, 3)


def run_sequential(seq: nn.Sequential, x_seq: torch.Tensor) -> torch.Tensor:
    """``seq(x_seq)`` with every eligible (convolution, batch norm, neuron) run of three modules executed fused."""
    mods = list(seq)
    i = 0
    while i < len(mods):
        if i + 2 < len(mods) and isinstance(mods[i], nn.Conv2d) and isinstance(mods[i + 1], nn.BatchNorm2d) \
                and isinstance(mods[i + 2], base.MemoryModule) and getattr(mods[i], "step_mode", "s") == "m" \
                and eligible(mods[i], mods[i + 1], mods[i + 2], x_seq):
            x_seq = conv_bn_lif(mods[i], mods[i + 1], mods[i + 2], x_seq)
            i += 3
        else:
            x_seq = mods[i](x_seq)
            i += 1
    return x_seq
