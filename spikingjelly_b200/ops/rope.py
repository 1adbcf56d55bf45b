"""Rotary position embedding fused with the split of a packed, head-major QKV projection (``csrc/rope_qkv.cu``)."""
from __future__ import annotations

import torch

from . import counters, require

__all__ = ["rope_qkv", "supports"]


class _RopeQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, offset):
        counters.bump("rope_qkv")
        ctx.save_for_backward(cos, sin)
        ctx.offset = offset
        return torch.ops.sjb200.rope_qkv_forward(qkv, cos, sin, offset)

    @staticmethod
    def backward(ctx, gq, gk, gv):
        cos, sin = ctx.saved_tensors
        counters.bump("rope_qkv")
        return torch.ops.sjb200.rope_qkv_backward(gq.contiguous(), gk.contiguous(), gv.contiguous(), cos, sin, ctx.offset), None, None, None


def supports(qkv: torch.Tensor, head_dim: int) -> bool:
    return qkv.is_cuda and qkv.dtype in (torch.bfloat16, torch.float16) and head_dim % 16 == 0


def rope_qkv(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, offset: int = 0):
    """``qkv``: ``[N, S, H, 3, D]`` contiguous 16-bit; ``cos`` / ``sin``: fp32 ``[>= S + offset, D]`` (half-split convention:
    pairs ``(i, i + D/2)``).  Returns ``q, k, v`` as contiguous ``[N, S, H, D]`` with q and k rotated."""
    require()
    return _RopeQKV.apply(qkv.contiguous(), cos, sin, int(offset))
