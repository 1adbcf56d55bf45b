"""Linear and convolution layers for spike inputs that keep the input for backward as bits instead of floats
(``cuda_kernel/spike_op.py:124-734`` of the reference: there the saved spike becomes ``bool`` through a CuPy kernel and the
backward goes through an inline C++ wrapper of ``at::convolution_backward``).

Two routes.  16-bit CUDA inputs whose shapes the tensor-core kernels take (2-D convolutions with channel counts that are
multiples of 64, linears with feature counts that are multiples of 8) run natively in all three passes: forward, data
gradient and weight gradient are the implicit-GEMM convolution (``ops/conv.py``) or the tcgen05 GEMM (``ops/gemm.py``), and
the saved spike input is kept as 1 bit per element and expanded by the bit-unpacking kernel right before the two backward
products.  Everything else goes through one generic autograd function: forward is the library operator, the spike input is
stored with :data:`tensor_cache.BOOL_TENSOR_CACHE` (bit-packed at ``configure.save_bool_spike_level == 1``), and backward
rebuilds it and differentiates the same operator with ``torch.autograd.grad``.  Inputs must be 0 / 1 valued; on CPU tensors
the plain operators run."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn.modules.utils import _pair, _single, _triple

from . import tensor_cache

__all__ = ["spike_linear", "spike_conv1d", "spike_conv2d", "spike_conv3d", "SpikeLinear", "SpikeConv1d", "SpikeConv2d", "SpikeConv3d",
           "cupy_spike_linear_forward", "cupy_spike_convolution_forward"]

_OPS = {0: F.linear, 1: F.conv1d, 2: F.conv2d, 3: F.conv3d}


def _native_dtype(spike: torch.Tensor):
    """The 16-bit compute dtype of this call (the input's own, or the CUDA autocast dtype), else None."""
    if not spike.is_cuda:
        return None
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        return dt if dt in (torch.bfloat16, torch.float16) else None
    return spike.dtype if spike.dtype in (torch.bfloat16, torch.float16) else None


class _SpikeConv2dNative(torch.autograd.Function):
    """Forward / dgrad / wgrad on the tensor cores; the spike input is saved as bits."""

    @staticmethod
    def forward(ctx, spike, weight, bias, stride, padding, dilation, dt):
        from ...ops import bitpack, counters
        x = spike.detach().to(dt).permute(0, 2, 3, 1).contiguous()                      # NHWC
        w_krsc = weight.detach().to(dtype=dt, memory_format=torch.channels_last).permute(0, 2, 3, 1).contiguous()
        counters.bump("conv_tcgen05")
        rows, _ = torch.ops.sjb200.conv2d_nhwc_forward(x, w_krsc, stride, padding, dilation, False)
        if bias is not None:
            rows = rows + bias.detach().to(dt)
        ctx.bits = bitpack.bit_spike_compress(x)
        ctx.xshape, ctx.geom, ctx.dt = x.shape, (stride, padding, dilation), dt
        ctx.wmeta = (tuple(weight.shape), weight.dtype, spike.dtype, None if bias is None else bias.dtype)
        ctx.save_for_backward(w_krsc)
        n, h, w_, _c = x.shape
        oh = (h + 2 * padding[0] - dilation[0] * (weight.shape[2] - 1) - 1) // stride[0] + 1
        ow = (w_ + 2 * padding[1] - dilation[1] * (weight.shape[3] - 1) - 1) // stride[1] + 1
        return rows.view(n, oh, ow, weight.shape[0]).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, grad_out):
        from ...ops import bitpack, counters
        (w_krsc,) = ctx.saved_tensors
        stride, padding, dilation = ctx.geom
        wshape, wdtype, sdtype, bdtype = ctx.wmeta
        gy = grad_out.to(ctx.dt).permute(0, 2, 3, 1).contiguous()
        gy = gy.view(-1, gy.shape[-1])
        gs = gw = gb = None
        if ctx.needs_input_grad[0]:
            counters.bump("conv_tcgen05")
            gx = torch.ops.sjb200.conv2d_nhwc_dgrad(gy, w_krsc, ctx.xshape[1], ctx.xshape[2], stride, padding)
            gs = gx.permute(0, 3, 1, 2).to(sdtype)
        if ctx.needs_input_grad[1]:
            x = bitpack.bit_spike_decompress(ctx.bits, ctx.xshape, ctx.dt)
            counters.bump("conv_tcgen05")
            g = torch.ops.sjb200.conv2d_nhwc_wgrad(x, gy, wshape[2], wshape[3], stride, padding, dilation)
            gw = g.permute(0, 3, 1, 2).to(wdtype)
        if bdtype is not None and ctx.needs_input_grad[2]:
            gb = gy.float().sum(0).to(bdtype)
        ctx.bits = None
        return gs, gw, gb, None, None, None, None


class _SpikeLinearNative(torch.autograd.Function):
    @staticmethod
    def forward(ctx, spike, weight, bias, dt):
        from ...ops import bitpack
        from ...ops import gemm as G
        x2d = spike.detach().to(dt).reshape(-1, spike.shape[-1]).contiguous()
        w = weight.detach().to(dt).contiguous()
        y = G.gemm(x2d, w)
        if bias is not None:
            y = y + bias.detach().to(dt)
        ctx.bits, ctx.xshape, ctx.dt = bitpack.bit_spike_compress(x2d), x2d.shape, dt
        ctx.meta = (spike.shape, spike.dtype, weight.dtype, None if bias is None else bias.dtype)
        ctx.save_for_backward(w)
        return y.view(*spike.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad_out):
        from ...ops import bitpack
        from ...ops import gemm as G
        (w,) = ctx.saved_tensors
        sshape, sdtype, wdtype, bdtype = ctx.meta
        gy = grad_out.to(ctx.dt).reshape(-1, grad_out.shape[-1]).contiguous()
        gs = gw = gb = None
        if ctx.needs_input_grad[0]:
            gs = G.gemm(gy, w, False, True).view(sshape).to(sdtype)
        if ctx.needs_input_grad[1]:
            x2d = bitpack.bit_spike_decompress(ctx.bits, ctx.xshape, ctx.dt)
            gw = G.gemm(gy, x2d, True, True, out_f32=True).to(wdtype)
        if bdtype is not None and ctx.needs_input_grad[2]:
            gb = gy.float().sum(0).to(bdtype)
        ctx.bits = None
        return gs, gw, gb, None


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
    dt = _native_dtype(spike)
    if dt is not None and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0:
        return _SpikeLinearNative.apply(spike, weight, bias, dt)
    return _SpikeOp.apply(0, spike, weight, bias)


def _conv(nd, tup, spike, weight, bias, stride, padding, dilation, groups):
    if not spike.is_cuda or isinstance(padding, str):
        return _OPS[nd](spike, weight, bias, stride, padding, dilation, groups)
    return _SpikeOp.apply(nd, spike, weight, bias, tuple(tup(stride)), tuple(tup(padding)), tuple(tup(dilation)), groups)


def spike_conv1d(spike, weight, bias=None, stride=1, padding="valid", dilation=1, groups=1):
    return _conv(1, _single, spike, weight, bias, stride, padding, dilation, groups)


def spike_conv2d(spike, weight, bias=None, stride=1, padding="valid", dilation=1, groups=1):
    dt = _native_dtype(spike)
    if dt is not None and not isinstance(padding, str) and spike.dim() == 4:
        from ...ops import conv as conv_ops
        st, pd, dl = _pair(stride), _pair(padding), _pair(dilation)
        if conv_ops.supports_shape(weight.shape[1], weight.shape[0], weight.shape[2:], st, pd, dl, groups):
            return _SpikeConv2dNative.apply(spike, weight, bias, list(st), list(pd), list(dl), dt)
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


def cupy_spike_linear_forward(spike: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """The reference's operator name for :func:`spike_linear` (the input is kept for backward as bits)."""
    return spike_linear(spike, weight, bias)


def cupy_spike_convolution_forward(spike: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], stride, padding, dilation,
                                   groups: int) -> torch.Tensor:
    """The reference's operator name for ``spike_conv1d / 2d / 3d``, chosen by the rank of ``spike``."""
    fn = {3: spike_conv1d, 4: spike_conv2d, 5: spike_conv3d}.get(spike.dim())
    if fn is None:
        raise ValueError(f"expected a 3-, 4- or 5-dimensional spike tensor, got {spike.dim()} dimensions")
    as_arg = lambda v: v if isinstance(v, (int, str)) else tuple(v)          # noqa: E731
    return fn(spike, weight, bias, as_arg(stride), as_arg(padding), as_arg(dilation), groups)


#: the reference records here why its inline C++ wrapper failed to build; this package has no such wrapper
cpp_wrapper_error = None
