"""Linear and convolution layers for spike inputs that keep the input for backward as bits instead of floats
(``cuda_kernel/spike_op.py:124-734`` of the reference: there the saved spike becomes ``bool`` through a CuPy kernel and the
backward goes through an inline C++ wrapper of ``at::convolution_backward``).

Here one autograd function covers all of them: forward is the library operator, the spike input is stored with
:data:`tensor_cache.BOOL_TENSOR_CACHE` (bit-packed by the native kernel at ``configure.save_bool_spike_level == 1``, 1/32 of an
fp32 tensor), and backward rebuilds it and differentiates the same operator with ``torch.autograd.grad``.  Inputs must be
0 / 1 valued; on CPU tensors the plain operators run."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn.modules.utils import _pair, _single, _triple

from . import tensor_cache

__all__ = ["spike_linear", "spike_conv1d", "spike_conv2d", "spike_conv3d", "SpikeLinear", "SpikeConv1d", "SpikeConv2d", "SpikeConv3d"]

_OPS = {0: F.linear, 1: F.conv1d, 2: F.conv2d, 3: F.conv3d}


class _SpikeOp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, nd, spike, weight, bias, *conv_args):
        op = _OPS[nd]
        out = op(spike, weight, bias, *conv_args)
        ctx.nd, ctx.conv_args, ctx.shape, ctx.spike_needs_grad = nd, conv_args, spike.shape, spike.requires_grad
        ctx.key = tensor_cache.BOOL_TENSOR_CACHE.store_bool(spike.detach())
        ctx.save_for_backward(weight, bias if bias is not None else weight.new_empty(0))
        ctx.has_bias = bias is not None
        return out

    @staticmethod
    def backward(ctx, grad_out):
        weight, bias = ctx.saved_tensors
        spike = tensor_cache.BOOL_TENSOR_CACHE.get_float(ctx.key, ctx.shape)
        with torch.enable_grad():
            s = spike.detach().requires_grad_(ctx.spike_needs_grad)
            w = weight.detach().requires_grad_(True)
            b = bias.detach().requires_grad_(True) if ctx.has_bias else None
            out = _OPS[ctx.nd](s, w, b, *ctx.conv_args)
            wanted = [t for t in (s if ctx.spike_needs_grad else None, w, b) if t is not None]
            grads = list(torch.autograd.grad(out, wanted, grad_out))
        gs = grads.pop(0) if ctx.spike_needs_grad else None
        gw = grads.pop(0)
        gb = grads.pop(0) if ctx.has_bias else None
        return (None, gs, gw, gb) + (None,) * len(ctx.conv_args)


def spike_linear(spike, weight, bias: Optional[torch.Tensor] = None):
    if not spike.is_cuda:
        return F.linear(spike, weight, bias)
    return _SpikeOp.apply(0, spike, weight, bias)


def _conv(nd, tup, spike, weight, bias, stride, padding, dilation, groups):
    if not spike.is_cuda or isinstance(padding, str):
        return _OPS[nd](spike, weight, bias, stride, padding, dilation, groups)
    return _SpikeOp.apply(nd, spike, weight, bias, tuple(tup(stride)), tuple(tup(padding)), tuple(tup(dilation)), groups)


def spike_conv1d(spike, weight, bias=None, stride=1, padding="valid", dilation=1, groups=1):
    return _conv(1, _single, spike, weight, bias, stride, padding, dilation, groups)


def spike_conv2d(spike, weight, bias=None, stride=1, padding="valid", dilation=1, groups=1):
    return _conv(2, _pair, spike, weight, bias, stride, padding, dilation, groups)


def spike_conv3d(spike, weight, bias=None, stride=1, padding="valid", dilation=1, groups=1):
    return _conv(3, _triple, spike, weight, bias, stride, padding, dilation, groups)


class SpikeLinear(nn.Linear):
    def forward(self, spike):
        return spike_linear(spike, self.weight, self.bias)


def _conv_module(base, fn, zero):
    class _SpikeConv(base):
        def _conv_forward(self, spike, weight, bias):
            if self.padding_mode != "zeros":
                spike = F.pad(spike, self._reversed_padding_repeated_twice, mode=self.padding_mode)
                return fn(spike, weight, bias, self.stride, zero(0), self.dilation, self.groups)
            return fn(spike, weight, bias, self.stride, self.padding, self.dilation, self.groups)
    return _SpikeConv


SpikeConv1d = _conv_module(nn.Conv1d, spike_conv1d, _single)
SpikeConv1d.__name__ = SpikeConv1d.__qualname__ = "SpikeConv1d"
SpikeConv2d = _conv_module(nn.Conv2d, spike_conv2d, _pair)
SpikeConv2d.__name__ = SpikeConv2d.__qualname__ = "SpikeConv2d"
SpikeConv3d = _conv_module(nn.Conv3d, spike_conv3d, _triple)
SpikeConv3d.__name__ = SpikeConv3d.__qualname__ = "SpikeConv3d"
