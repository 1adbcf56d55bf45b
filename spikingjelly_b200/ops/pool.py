"""Channels-last 3 x 3 / stride 2 / padding 1 max pooling with a one-byte argmax code (``csrc/pool_nhwc.cu``).

The spiking ResNet stems pool spike maps ``[T * B, C, H, W]`` held channels-last; the library NHWC max-pool kernels
run far below the copy rate there (backward scatters with 64-bit indices).  Here forward writes the window
maximum and ``kh * 3 + kw`` of its first occurrence, and backward lets every input pixel gather from the (at most four)
windows that cover it, so each gradient element is written exactly once."""
from __future__ import annotations

import torch

from . import counters, require

__all__ = ["max_pool_3x3s2_channels_last", "supports"]


class _MaxPool3x3S2(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_nhwc):
        counters.bump("maxpool_nhwc")
        out, idx = torch.ops.sjb200.maxpool3x3s2_nhwc_forward(x_nhwc)
        ctx.save_for_backward(idx)
        ctx.hw = (x_nhwc.shape[1], x_nhwc.shape[2])
        return out

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        counters.bump("maxpool_nhwc")
        return torch.ops.sjb200.maxpool3x3s2_nhwc_backward(g.contiguous(), idx, ctx.hw[0], ctx.hw[1])


def supports(pool: torch.nn.Module, x: torch.Tensor) -> bool:
    """True when ``pool`` is MaxPool2d(3, 2, 1) without dilation / ceil mode and ``x`` is a 16-bit CUDA tensor
    ``[N, C, H, W]`` stored channels-last with ``C % 8 == 0``."""
    def _pair(v):
        return tuple(v) if isinstance(v, (tuple, list)) else (v, v)
    if not isinstance(pool, torch.nn.MaxPool2d) or pool.return_indices or pool.ceil_mode:
        return False
    if _pair(pool.kernel_size) != (3, 3) or _pair(pool.stride) != (2, 2) or _pair(pool.padding) != (1, 1) or _pair(pool.dilation) != (1, 1):
        return False
    return (x.is_cuda and x.dim() == 4 and x.dtype in (torch.bfloat16, torch.float16) and x.shape[1] % 8 == 0
            and x.is_contiguous(memory_format=torch.channels_last))


def max_pool_3x3s2_channels_last(x: torch.Tensor) -> torch.Tensor:
    """``x``: ``[N, C, H, W]`` with channels-last strides -> ``[N, C, OH, OW]`` with channels-last strides."""
    require()
    y = _MaxPool3x3S2.apply(x.permute(0, 2, 3, 1))          # a view: NHWC is how the bytes already lie
    return y.permute(0, 3, 1, 2)
