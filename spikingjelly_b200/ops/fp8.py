"""fp8 (e4m3 / e5m2) tensor-core linear algebra with per-tensor dynamic scaling.

``quantize(x)`` -> ``(q, inv_scale)`` with ``x ~= q.float() * inv_scale``; ``matmul_nt(a_q, b_q, alpha)``
computes ``alpha * a_q @ b_q.T`` on the tcgen05 tensor cores (``kind::f8f6f4``, fp32 accumulation in
TMEM) and returns bf16; ``linear(x, weight, bias)`` is the differentiable layer built from them:

* forward  ``y = x W^T``        fp8 x fp8   (x: e4m3, W: e4m3)
* dgrad    ``dx = dy W``        fp8 x fp8   (dy: e5m2 - gradients need range more than precision)
* wgrad    ``dW = dy^T x``      bf16 x bf16 on the 16-bit kernel (operands are token-major, which the
  8-bit tensor-core path cannot contract over); ``x`` is kept for backward as fp8 bytes — exact for
  spikes — and widened on the fly.

Binary spike inputs are exactly representable in e4m3, so only weights and gradients lose precision.
On machines without CUDA the same functions run through PyTorch ops on de-quantised values.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

__all__ = ["quantize", "dequantize", "matmul_nt", "linear", "E4M3_MAX", "E5M2_MAX"]

E4M3_MAX, E5M2_MAX = 448.0, 57344.0


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda


def quantize(x: torch.Tensor, e5m2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-tensor dynamic quantisation: ``scale = max_repr / amax(x)``; returns ``(q, 1 / scale)``."""
    if _native(x) and x.dtype in (torch.float32, torch.float16, torch.bfloat16):
        from . import counters, require
        require()
        counters.bump("fp8_quantize", 2)
        return torch.ops.sjb200.fp8_quantize(x, e5m2)
    fmax = E5M2_MAX if e5m2 else E4M3_MAX
    amax = x.detach().abs().amax().float()
    scale = torch.where(amax > 0, fmax / amax, torch.ones_like(amax))
    q = (x.float() * scale).clamp(-fmax, fmax).to(torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn)
    return q, (1.0 / scale).reshape(1)


def dequantize(q: torch.Tensor, inv_scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    return (q.to(torch.float32) * inv_scale).to(dtype)


def matmul_nt(a_q: torch.Tensor, b_q: torch.Tensor, alpha: Optional[torch.Tensor] = None, out_f32: bool = False) -> torch.Tensor:
    """``alpha * a_q [M, K] @ b_q [N, K]^T`` -> bf16 (or fp32) ``[M, N]``."""
    if _native(a_q):
        from . import counters, require
        require()
        counters.bump("gemm_fp8")
        return torch.ops.sjb200.gemm_fp8(a_q, b_q, alpha, out_f32, 0)
    y = a_q.float() @ b_q.float().t()
    if alpha is not None:
        y = y * alpha
    return y if out_f32 else y.to(torch.bfloat16)


class _Fp8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, weight, bias):
        xq, sx = quantize(x2d)
        wq, sw = quantize(weight)
        y = matmul_nt(xq, wq, sx * sw)
        if bias is not None:
            y = y + bias.to(y.dtype)
        ctx.save_for_backward(xq, sx, weight)
        ctx.has_bias = bias is not None
        ctx.in_dtype = x2d.dtype
        return y.to(x2d.dtype) if x2d.dtype != torch.float32 else y.float()

    @staticmethod
    def backward(ctx, gy):
        xq, sx, weight = ctx.saved_tensors
        gy = gy.contiguous()
        gx = gw = gb = None
        g16 = gy.to(torch.bfloat16)
        if ctx.needs_input_grad[0]:
            gq, sg = quantize(g16, e5m2=True)
            # e5m2 x e5m2: the kernel takes one format for both operands
            wtq, swt = quantize(weight.t().contiguous(), e5m2=True)
            gx = matmul_nt(gq, wtq, sg * swt).to(ctx.in_dtype)
        if ctx.needs_input_grad[1]:
            x16 = dequantize(xq, sx)
            if _native(g16):
                from . import gemm as G
                gw = G.gemm(g16, x16, a_mn=True, b_mn=True, out_f32=True)       # dy^T x, contraction over tokens
            else:
                gw = g16.float().t() @ x16.float()
            gw = gw.to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = gy.float().sum(0)
        return gx, gw, gb


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp8 ``F.linear``: any leading dimensions; ``in_features`` must be a multiple of 16 and
    ``out_features`` of 8 (tensor-core tile constraints), otherwise falls back to ``F.linear``."""
    k, n = weight.shape[1], weight.shape[0]
    if k % 16 or n % 16:
        return torch.nn.functional.linear(x, weight, bias)
    y = _Fp8Linear.apply(x.reshape(-1, k), weight, bias)
    return y.reshape(*x.shape[:-1], n)
