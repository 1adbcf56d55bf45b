"""Spiking self-attention core ``O = scale * Q (K^T V)`` as one kernel per direction."""
from __future__ import annotations

import torch

from . import counters, require

__all__ = ["ssa"]


class _SSA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, S, L: int, heads: int, scale: float):
        counters.bump("ssa_forward")
        ctx.save_for_backward(S)
        ctx.L, ctx.heads, ctx.scale = L, heads, scale
        return torch.ops.sjb200.ssa_forward(S, L, heads, scale)

    @staticmethod
    def backward(ctx, dO):
        (S,) = ctx.saved_tensors
        counters.bump("ssa_backward")
        return torch.ops.sjb200.ssa_backward(dO.contiguous(), S, ctx.L, ctx.heads, ctx.scale), None, None, None


def ssa(S: torch.Tensor, L: int, heads: int, scale: float) -> torch.Tensor:
    """``S``: contiguous ``[..., L, 3*C]`` holding q, k, v (each ``C = heads * head_dim`` channels,
    head-major); returns ``[..., L, C]``.  ``head_dim`` must be 32 or 64, dtype bf16/fp16."""
    require()
    return _SSA.apply(S.contiguous(), int(L), int(heads), float(scale))
