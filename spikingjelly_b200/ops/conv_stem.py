"""Convolution with very few input channels (network stems: 2 polarity channels, RGB) as patch matrix + tensor-core GEMM.

``conv2d_few_channels(x, weight, stride, padding)`` takes a channels-last ``[N, C_in, H, W]`` activation that needs no
gradient (the network input) and returns ``(y_rows [N * OH * OW, C_out], stats, (OH, OW))``: the rows ARE the channels-last
output, and ``stats`` are the per-channel sums for the batch norm that follows (from the GEMM epilogue).  Backward is
one GEMM for the weight gradient over the saved patch matrix.  cuDNN pads C_in to 8 and runs these layers at a
fraction of the memory rate; see ``csrc/im2col_nhwc.cu``."""
from __future__ import annotations

from typing import Tuple

import torch

from . import counters, require
from . import gemm as G

__all__ = ["conv2d_few_channels", "supports"]


def _pair(v) -> Tuple[int, int]:
    return (int(v[0]), int(v[1])) if isinstance(v, (tuple, list)) else (int(v), int(v))


def supports(conv: torch.nn.Conv2d, x: torch.Tensor) -> bool:
    return (isinstance(conv, torch.nn.Conv2d) and conv.groups == 1 and _pair(conv.dilation) == (1, 1) and conv.bias is None
            and conv.padding_mode == "zeros" and not isinstance(conv.padding, str) and conv.in_channels <= 4
            and conv.out_channels % 8 == 0 and x.is_cuda and x.dim() == 4 and not x.requires_grad
            and x.dtype in (torch.bfloat16, torch.float16) and x.is_contiguous(memory_format=torch.channels_last))


class _ConvFewChannels(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_nhwc, weight, stride, padding, want_stats):
        co, ci, kh, kw = weight.shape
        counters.bump("im2col_nhwc")
        A = torch.ops.sjb200.im2col_nhwc(x_nhwc, kh, kw, stride[0], stride[1], padding[0], padding[1])
        K, Kp = kh * kw * ci, A.shape[1]
        w2 = weight.permute(0, 2, 3, 1).reshape(co, K).to(A.dtype)              # (kh, kw, c) order, like the patch columns
        if Kp != K:
            w2 = torch.nn.functional.pad(w2, (0, Kp - K))
        counters.bump("gemm_tcgen05")
        if want_stats:
            y, stats = torch.ops.sjb200.gemm_16bit_stats(A, w2.contiguous(), False, False)
        else:
            y, stats = torch.ops.sjb200.gemm_16bit(A, w2.contiguous(), False, False, False, 0), A.new_empty(0, dtype=torch.float32)
        ctx.save_for_backward(A)
        ctx.wshape = (co, ci, kh, kw)
        ctx.wdtype = weight.dtype
        ctx.mark_non_differentiable(stats)
        return y, stats

    @staticmethod
    def backward(ctx, gy, _gs):
        (A,) = ctx.saved_tensors
        co, ci, kh, kw = ctx.wshape
        gw2 = G.gemm(gy.contiguous(), A, True, True)                                 # [co, Kp] = gy^T A
        gw = gw2[:, :kh * kw * ci].reshape(co, kh, kw, ci).permute(0, 3, 1, 2).to(ctx.wdtype)
        return None, gw, None, None, None


def conv2d_few_channels(x: torch.Tensor, weight: torch.Tensor, stride, padding, want_stats: bool = True):
    """``x``: ``[N, C_in, H, W]`` channels-last, 16-bit, no gradient.  Returns ``(rows [N*OH*OW, C_out], stats or None, (OH, OW))``."""
    require()
    stride, padding = _pair(stride), _pair(padding)
    kh, kw = weight.shape[2], weight.shape[3]
    oh = (x.shape[2] + 2 * padding[0] - kh) // stride[0] + 1
    ow = (x.shape[3] + 2 * padding[1] - kw) // stride[1] + 1
    y, stats = _ConvFewChannels.apply(x.permute(0, 2, 3, 1), weight, stride, padding, want_stats)
    return y, (stats if want_stats else None), (oh, ow)
