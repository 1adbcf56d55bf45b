"""Fused parallel-spiking-neuron operator: ``S = (W X + b >= 0)`` over the time axis in one kernel
(``ops/csrc/psn.cu``).  The pre-activation ``H = W X + b`` is never written: forward reads ``X`` and writes the spikes,
backward recomputes ``H`` from ``X`` in registers.  ``W`` is any ``[T, T]`` matrix, so the masked and the sliding variants
use the same operator with their effective matrix, and their own parameters get their gradients through ordinary autograd
on that matrix."""
from __future__ import annotations

from typing import Tuple

import torch

__all__ = ["psn_spikes", "supported"]

MAX_T = 32


def supported(x_seq: torch.Tensor, spec) -> bool:
    """CUDA, fp32 / fp16 / bf16, ``T <= 32``, 16-byte aligned rows and a surrogate with a kernel descriptor."""
    if spec is None or not (torch.is_tensor(x_seq) and x_seq.is_cuda) or x_seq.dim() < 2:
        return False
    if x_seq.dtype not in (torch.float32, torch.float16, torch.bfloat16) or not 1 <= x_seq.shape[0] <= MAX_T:
        return False
    n = x_seq[0].numel()
    return n > 0 and n % (16 // x_seq.element_size()) == 0


class _PSN(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_seq, weight, bias, spec, sg):
        from . import counters
        x = x_seq.contiguous()
        w, b = weight.detach().float().contiguous(), bias.detach().float().reshape(-1).contiguous()
        counters.bump("psn_forward")
        s = torch.ops.sjb200.psn_forward(x, w, b)
        ctx.save_for_backward(x, w, b)
        ctx.spec, ctx.sg, ctx.dtypes = spec, sg, (weight.dtype, bias.dtype, bias.shape)
        return s

    @staticmethod
    def backward(ctx, grad_s):
        from . import counters
        x, w, b = ctx.saved_tensors
        counters.bump("psn_backward")
        T = x.shape[0]
        if T <= 8:
            # weight and bias gradients come out of the same kernel (per-block partial sums added in a fixed order)
            gx, gw, gb = torch.ops.sjb200.psn_backward_small(x, grad_s.contiguous().to(x.dtype), w, b, int(ctx.spec[0]), float(ctx.spec[1]), float(ctx.spec[2]))
            return ((gx if ctx.needs_input_grad[0] else None), gw.to(ctx.dtypes[0]) if ctx.needs_input_grad[1] else None,
                    gb.to(ctx.dtypes[1]).view(ctx.dtypes[2]) if ctx.needs_input_grad[2] else None, None, None)
        if ctx.sg is not None:
            # long time axes: T x T products per column exceed what one thread holds; recompute H with the library GEMM
            # (still nothing but X was kept since forward) and differentiate the surrogate through PyTorch
            x2 = x.view(T, -1)
            with torch.enable_grad():
                h = torch.addmm(b.view(-1, 1).to(x.dtype), w.to(x.dtype), x2).requires_grad_(True)
                (gh,) = torch.autograd.grad(ctx.sg(h), h, grad_s.reshape(T, -1).to(x.dtype))
            gx = torch.mm(w.to(x.dtype).t(), gh).view(x.shape) if ctx.needs_input_grad[0] else None
            gw = torch.mm(gh, x2.t()).to(ctx.dtypes[0]) if ctx.needs_input_grad[1] else None
            gb = gh.sum(1, dtype=torch.float32).to(ctx.dtypes[1]).view(ctx.dtypes[2]) if ctx.needs_input_grad[2] else None
            return gx, gw, gb, None, None
        gx, gh = torch.ops.sjb200.psn_backward(x, grad_s.contiguous().to(x.dtype), w, b, int(ctx.spec[0]), float(ctx.spec[1]), float(ctx.spec[2]))
        gw = gb = None
        if ctx.needs_input_grad[1]:
            # dW = dH X^T: a [T, T] result over a very long contraction; cut it into batched pieces of moderate depth
            n = x[0].numel()
            pieces = next((c for c in (1024, 512, 256, 128, 64) if n % c == 0 and n // c >= 1024), 1)
            a, c = gh.view(T, pieces, -1).transpose(0, 1), x.view(T, pieces, -1).permute(1, 2, 0)
            gw = torch.bmm(a, c).sum(0, dtype=torch.float32).to(ctx.dtypes[0])
        if ctx.needs_input_grad[2]:
            gb = gh.view(T, -1).sum(1, dtype=torch.float32).to(ctx.dtypes[1]).view(ctx.dtypes[2])
        return (gx if ctx.needs_input_grad[0] else None), gw, gb, None, None


def psn_spikes(x_seq: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, spec: Tuple[int, float, float], sg=None) -> torch.Tensor:
    """Spikes of shape ``x_seq.shape``; ``weight`` ``[T, T]``, ``bias`` ``[T, 1]`` or ``[T]``; ``spec`` the surrogate's
    ``(id, p0, p1)``.  Differentiable in all three tensors.  Forward is always the fused kernel.  Backward is the fused
    kernel for ``T <= 8`` (measured 1.8 - 11x the eager path); for longer time axes it recomputes ``H`` with the library
    GEMM when the surrogate module ``sg`` is given (the fused T x T recurrence per column is slower there), else it uses
    the general fused kernel."""
    from . import require
    require()
    return _PSN.apply(x_seq, weight, bias, spec, sg)
