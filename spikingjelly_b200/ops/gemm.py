"""tcgen05 GEMM front end: ``linear`` with autograd (forward, dgrad and wgrad all run in
the same persistent TMA/TMEM kernel; operands are consumed in place, including the
"transposed" ones, so no transpose is materialised)."""
from __future__ import annotations

from typing import Optional

import torch

from . import counters, require

__all__ = ["gemm", "linear", "linear_with_stats", "check_status"]


def gemm(a: torch.Tensor, b: torch.Tensor, a_mn: bool = False, b_mn: bool = False, out_f32: bool = False,
         split_k: int = 0) -> torch.Tensor:
    """``D[M, N] = sum_k A[m, k] B[n, k]`` with fp32 accumulation.

    ``a`` is ``[M, K]`` (``a_mn=False``) or ``[K, M]`` (``a_mn=True``); ``b`` is ``[N, K]`` or
    ``[K, N]`` likewise.  bf16 or fp16 operands; ``N`` and the leading dimensions must be
    multiples of 8."""
    require()
    counters.bump("gemm_tcgen05")
    return torch.ops.sjb200.gemm_16bit(a, b, a_mn, b_mn, out_f32, split_k)


def check_status(like: torch.Tensor) -> None:
    """Raise if a bounded wait inside a GEMM launched on ``like``'s device gave up."""
    code, block, detail = torch.ops.sjb200.gemm_status(like)
    if code != 0:
        names = {1: "operand tile never arrived", 2: "smem stage never released",
                 3: "accumulator never completed", 4: "accumulator never drained"}
        raise RuntimeError(f"tcgen05 GEMM gave up waiting ({names.get(code, code)}) in block {block}, detail {detail}")


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, weight):
        ctx.save_for_backward(x2d, weight)
        return gemm(x2d, weight)

    @staticmethod
    def backward(ctx, gy):
        x2d, weight = ctx.saved_tensors
        gy = gy.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = gemm(gy, weight, False, True)                 # [M, N] x [N, K] -> [M, K]
        if ctx.needs_input_grad[1]:
            gw = gemm(gy, x2d, True, True, out_f32=False)      # [M, N]^T x [M, K] -> [N, K]
        return gx, gw


class _LinearStats(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, weight):
        ctx.save_for_backward(x2d, weight)
        require()
        counters.bump("gemm_tcgen05")
        y, stats = torch.ops.sjb200.gemm_16bit_stats(x2d, weight, False, False)
        ctx.mark_non_differentiable(stats)
        return y, stats

    @staticmethod
    def backward(ctx, gy, _gstats):
        return _Linear.backward(ctx, gy)


def linear_with_stats(x2d: torch.Tensor, weight: torch.Tensor):
    """``(x2d @ weight.T, partial)`` where ``partial[b, 0 | 1, n]`` is the sum | sum of squares of rows
    ``32 b .. 32 b + 31`` of the (rounded) result: the batch-norm statistics come out of the GEMM's epilogue
    instead of a second pass over the output.  Pass ``partial`` to ``ops.bn_lif.bn_lif(..., stats=partial)``."""
    return _LinearStats.apply(x2d, weight)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` over the last axis of ``x`` on the tensor cores.
    ``x`` and ``weight`` must share a 16-bit dtype; feature sizes multiples of 8."""
    lead = x.shape[:-1]
    y = _Linear.apply(x.reshape(-1, x.shape[-1]), weight)
    if bias is not None:
        y = y + bias
    return y.reshape(*lead, weight.shape[0])
