"""Channels-last 2-D convolution on the tensor cores (implicit GEMM, ``csrc/conv_tcgen05.cu``).

``conv2d_rows(x_nhwc, weight, stride, padding, dilation, want_stats)`` takes a contiguous ``[N, H, W, C_in]``
16-bit activation and the module's ``[C_out, C_in, R, S]`` weight (any dtype / layout) and returns
``(rows [N*OH*OW, C_out], stats or None, (OH, OW))``: ``rows`` IS the channels-last output, ``stats`` are the
per-channel partial sums a following batch norm needs (computed in the GEMM epilogue).  Forward, data gradient
and weight gradient all run in the persistent TMA / tcgen05 kernel; the patch matrix is never written out (the TMA
unit gathers it).  Plays the role of the reference's spike convolution
(``spikingjelly/activation_based/cuda_kernel/spike_op.py:34-62,124-256``) without a library convolution on either
pass.

``supports(conv, x)`` tells whether a layer can take this path: channel counts that are multiples of 64, groups 1,
zero padding, dilation 1; everything else stays with the caller's fallback.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import counters, require

__all__ = ["conv2d_rows", "conv2d_channels_last", "supports", "supports_shape"]


def _pair(v) -> Tuple[int, int]:
    return (int(v[0]), int(v[1])) if isinstance(v, (tuple, list)) else (int(v), int(v))


def supports_shape(c_in: int, c_out: int, kernel, stride, padding, dilation=(1, 1), groups: int = 1) -> bool:
    kh, kw = _pair(kernel)
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    return (groups == 1 and _pair(dilation) == (1, 1) and c_in % 64 == 0 and c_out % 64 == 0 and 1 <= sh <= 8 and 1 <= sw <= 8
            and kh <= 16 and kw <= 16 and 0 <= ph < 64 and 0 <= pw < 64)


def supports(conv: torch.nn.Conv2d, x: torch.Tensor) -> bool:
    """``x``: the ``[N, C, H, W]``-shaped (channels-last) activation that ``conv`` is about to see."""
    return (isinstance(conv, torch.nn.Conv2d) and conv.padding_mode == "zeros" and not isinstance(conv.padding, str)
            and supports_shape(conv.in_channels, conv.out_channels, conv.kernel_size, conv.stride, conv.padding, conv.dilation, conv.groups)
            and x.is_cuda and x.dim() == 4 and x.dtype in (torch.bfloat16, torch.float16))


class _ConvRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_nhwc, weight, stride, padding, dilation, want_stats):
        # [C_out, C_in, R, S] -> the memory of its channels-last form, [C_out, R, S, C_in], in the compute dtype
        w_krsc = weight.detach().to(dtype=x_nhwc.dtype, memory_format=torch.channels_last).permute(0, 2, 3, 1)
        if not w_krsc.is_contiguous():          # 1 x 1 filters: channels-last and contiguous strides coincide ambiguously
            w_krsc = w_krsc.contiguous()
        counters.bump("conv_tcgen05")
        y, stats = torch.ops.sjb200.conv2d_nhwc_forward(x_nhwc, w_krsc, stride, padding, dilation, want_stats)
        ctx.save_for_backward(x_nhwc, w_krsc)
        ctx.geom = (stride, padding, dilation, tuple(weight.shape), weight.dtype)
        ctx.mark_non_differentiable(stats)
        return y, stats

    @staticmethod
    def backward(ctx, gy, _gstats):
        x_nhwc, w_krsc = ctx.saved_tensors
        stride, padding, dilation, wshape, wdtype = ctx.geom
        gy = gy.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            counters.bump("conv_tcgen05")
            gx = torch.ops.sjb200.conv2d_nhwc_dgrad(gy, w_krsc, x_nhwc.shape[1], x_nhwc.shape[2], stride, padding)
        if ctx.needs_input_grad[1]:
            counters.bump("conv_tcgen05")
            g = torch.ops.sjb200.conv2d_nhwc_wgrad(x_nhwc, gy, wshape[2], wshape[3], stride, padding, dilation)
            gw = g.permute(0, 3, 1, 2).to(wdtype)          # [C_out, C_in, R, S] view of channels-last memory
        return gx, gw, None, None, None, None


def conv2d_rows(x_nhwc: torch.Tensor, weight: torch.Tensor, stride=1, padding=0, dilation=1, want_stats: bool = False):
    """``x_nhwc``: contiguous ``[N, H, W, C_in]``, bf16 / fp16.  Returns ``(rows [N*OH*OW, C_out], stats | None, (OH, OW))``."""
    require()
    stride, padding, dilation = list(_pair(stride)), list(_pair(padding)), list(_pair(dilation))
    if not x_nhwc.is_contiguous():
        x_nhwc = x_nhwc.contiguous()
    kh, kw = weight.shape[2], weight.shape[3]
    oh = (x_nhwc.shape[1] + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    ow = (x_nhwc.shape[2] + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    y, stats = _ConvRows.apply(x_nhwc, weight, stride, padding, dilation, want_stats)
    return y, (stats if want_stats else None), (oh, ow)


def conv2d_channels_last(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, stride=1, padding=0,
                         dilation=1) -> torch.Tensor:
    """Drop-in for ``F.conv2d`` on an ``[N, C, H, W]``-shaped tensor: the result is ``[N, C_out, OH, OW]``-shaped
    channels-last memory.  The input is brought to channels-last first if it is not."""
    nhwc = x.permute(0, 2, 3, 1)
    rows, _, (oh, ow) = conv2d_rows(nhwc, weight, stride, padding, dilation)
    if bias is not None:
        rows = rows + bias.to(rows.dtype)
    return rows.view(x.shape[0], oh, ow, weight.shape[0]).permute(0, 3, 1, 2)
