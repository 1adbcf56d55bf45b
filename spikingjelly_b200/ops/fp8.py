"""fp8 (e4m3 / e5m2) tensor-core linear algebra with per-tensor scaling, current or delayed.

``quantize(x)`` -> ``(q, inv_scale)`` with ``x ~= q.float() * inv_scale``; ``matmul_nt(a_q, b_q, alpha)``
computes ``alpha * a_q @ b_q.T`` on the tcgen05 tensor cores (``kind::f8f6f4``, fp32 accumulation in
TMEM) and returns bf16; ``linear(x, weight, bias, scaling)`` is the differentiable layer built from them:

* forward  ``y = x W^T``        x: e4m3, W: e4m3
* dgrad    ``dx = dy W``        dy: e5m2 (gradients need range more than precision), W^T: e4m3
* wgrad    ``dW = dy^T x``      dy^T: e5m2, x^T: e4m3, fp32 result

Every tensor is read once: the quantising kernel writes the row-major and the transposed bytes together, and with
delayed scaling (:class:`LinearScaling`) it takes the scale from the previous call and records the maximum for the
next one in the same pass.  What backward keeps of ``x`` is its transposed fp8 copy, one byte per element.

Binary spike inputs are exactly representable in e4m3, so only weights and gradients lose precision.
On machines without CUDA the same functions run through PyTorch ops on de-quantised values.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

__all__ = ["quantize", "quantize_with", "dequantize", "matmul_nt", "linear", "ScalingState", "LinearScaling", "E4M3_MAX", "E5M2_MAX"]

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
    scale = torch.where(amax > 0, torch.full_like(amax, fmax) / amax, torch.ones_like(amax))
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


class ScalingState:
    """Delayed-scaling state of one tensor role (a layer's input, weight or output gradient): three maxima used in
    rotation, so that each call scales with the maximum recorded by the call before it while recording its own (the
    kernel in ``ops/csrc/fp8_cast.cu`` does both in the single pass over the data).  The first call has no history and
    scales by the tensor's own maximum."""

    def __init__(self):
        self.amax3: Optional[torch.Tensor] = None
        self.calls = 0

    def _ready(self, x: torch.Tensor) -> bool:
        if self.amax3 is None or self.amax3.device != x.device:
            self.amax3 = torch.zeros(3, dtype=torch.float32, device=x.device)
            self.calls = 0
        return self.calls > 0

    def _seed(self, inv_scale: torch.Tensor, fmax: float) -> None:
        # the first call ran with its own maximum: amax = fmax * inv_scale
        self.amax3[0] = inv_scale.reshape(()) * fmax
        self.calls = 1


def _quantize_reference(x, fmax, f8, amax):
    # tensor / tensor is a true division like the kernel's; ``float / tensor`` would be reciprocal-times-scalar, one ulp off
    scale = torch.where(amax > 0, torch.full_like(amax, fmax) / amax, torch.ones_like(amax))
    return (x.float() * scale).clamp(-fmax, fmax).to(f8), (1.0 / scale).reshape(1)


def quantize_with(x: torch.Tensor, state: Optional[ScalingState], e5m2: bool = False,
                  transpose: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor]:
    """``(q, q_transposed or None, inv_scale)`` of ``x``.  ``state=None``: scale by the tensor's own maximum (two
    passes); otherwise delayed scaling on ``state`` (one pass).  ``transpose=True`` also returns ``q.T`` as a
    contiguous matrix; on CUDA it comes out of the same pass when ``x`` is a 16-bit ``[R, C]`` matrix with ``R % 64 ==
    0`` and ``C % 128 == 0``."""
    fmax = E5M2_MAX if e5m2 else E4M3_MAX
    f8 = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    delayed = state is not None and state._ready(x)
    if _native(x) and x.dtype in (torch.float32, torch.float16, torch.bfloat16):
        from . import counters, require
        require()
        fused_t = transpose and x.dim() == 2 and x.dtype != torch.float32 and x.shape[0] % 64 == 0 and x.shape[1] % 128 == 0
        if fused_t:
            counters.bump("fp8_quantize", 1 if delayed else 2)
            q, qt, inv = torch.ops.sjb200.fp8_quantize_transpose(x, state.amax3 if delayed else None, state.calls if delayed else 0, e5m2)
        else:
            if delayed:
                counters.bump("fp8_quantize")
                q, inv = torch.ops.sjb200.fp8_quantize_delayed(x, state.amax3, state.calls, e5m2)
            else:
                counters.bump("fp8_quantize", 2)
                q, inv = torch.ops.sjb200.fp8_quantize(x, e5m2)
            qt = q.t().contiguous() if transpose else None
    else:
        xd = x.detach()
        cur = xd.abs().amax().float() if xd.numel() else xd.new_zeros((), dtype=torch.float32)
        if delayed:
            k = state.calls
            q, inv = _quantize_reference(xd, fmax, f8, state.amax3[(k + 2) % 3])
            state.amax3[k % 3] = torch.maximum(state.amax3[k % 3], cur)
            state.amax3[(k + 1) % 3] = 0.0
        else:
            q, inv = _quantize_reference(xd, fmax, f8, cur)
        qt = q.t().contiguous() if transpose else None
    if state is not None:
        if delayed:
            state.calls += 1
        else:
            state._seed(inv, fmax)
    return q, qt, inv


class LinearScaling:
    """Per-layer state of an fp8 linear: the three tensor roles under delayed scaling (``delayed=False``: every tensor
    is scaled by its own maximum and only the weight cache below is used), and the quantised weight of the last
    gradient-free call, reused while the parameter has not been written (inference quantises the weight once)."""

    def __init__(self, delayed: bool = True):
        self.delayed = bool(delayed)
        self.x, self.w, self.g = ScalingState(), ScalingState(), ScalingState()
        self._frozen = None                 # (data_ptr, version, wq, inv_scale)

    def role(self, name: str) -> Optional[ScalingState]:
        return getattr(self, name) if self.delayed else None

    def frozen_weight(self, weight: torch.Tensor):
        key = (weight.data_ptr(), weight._version)
        if self._frozen is None or self._frozen[0] != key:
            w16 = weight.detach() if weight.dtype in (torch.bfloat16, torch.float16) else weight.detach().to(torch.bfloat16)
            wq, _, sw = quantize_with(w16, None)
            self._frozen = (key, wq, sw)
        return self._frozen[1], self._frozen[2]


def _mm(a_q, b_q, sa, sb, out_f32=False, bias=None):
    """``sa * sb * a_q @ b_q.T (+ bias)``; scales and bias are applied in the GEMM epilogue."""
    if _native(a_q):
        from . import counters, require
        require()
        counters.bump("gemm_fp8")
        return torch.ops.sjb200.gemm_fp8(a_q, b_q, sa, out_f32, 0, sb, bias)
    y = (a_q.float() @ b_q.float().t()) * (sa * sb)
    if bias is not None:
        y = y + bias.float()
    return y if out_f32 else y.to(torch.bfloat16)


def _result_dtype(x: torch.Tensor) -> torch.dtype:
    """What ``F.linear`` would return for this input: the autocast dtype inside an autocast region, else the input's."""
    if torch.is_autocast_enabled(x.device.type):
        return torch.get_autocast_dtype(x.device.type)
    return x.dtype


def _as(y: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return y if y.dtype == dtype else y.to(dtype)


class _Fp8Linear(torch.autograd.Function):
    """All three products on the 8-bit tensor cores.  Each of x, W and dy is quantised once, in a pass that also
    writes the transposed bytes, because forward (x W^T), data gradient (dy W) and weight gradient (dy^T x) contract
    over features-in, features-out and tokens respectively.  x and W are e4m3, dy is e5m2 (the GEMM mixes formats)."""

    @staticmethod
    def forward(ctx, x2d, weight, bias, scaling):
        need_gw, need_gx = weight.requires_grad, x2d.requires_grad
        x16 = x2d if x2d.dtype in (torch.bfloat16, torch.float16) else x2d.to(torch.bfloat16)
        w16 = weight.detach() if weight.dtype in (torch.bfloat16, torch.float16) else weight.detach().to(torch.bfloat16)
        xq, xqt, sx = quantize_with(x16, scaling.role("x") if scaling else None, transpose=need_gw)
        wq, wqt, sw = quantize_with(w16, scaling.role("w") if scaling else None, transpose=need_gx)
        y = _mm(xq, wq, sx, sw, bias=None if bias is None else bias.detach())
        ctx.save_for_backward(xqt, sx, wqt, sw)
        ctx.scaling, ctx.has_bias, ctx.in_dtype, ctx.w_dtype = scaling, bias is not None, x2d.dtype, weight.dtype
        return _as(y, _result_dtype(x2d))

    @staticmethod
    def backward(ctx, gy):
        xqt, sx, wqt, sw = ctx.saved_tensors
        gx = gw = gb = None
        g16 = gy.contiguous()
        if g16.dtype not in (torch.bfloat16, torch.float16):
            g16 = g16.to(torch.bfloat16)
        need_gx, need_gw = ctx.needs_input_grad[0] and wqt is not None, ctx.needs_input_grad[1] and xqt is not None
        gq, gqt, sg = quantize_with(g16, ctx.scaling.role("g") if ctx.scaling else None, e5m2=True, transpose=need_gw)
        if need_gx:
            gx = _mm(gq, wqt, sg, sw).to(ctx.in_dtype)                 # [M, N] x [K, N]^T
        if need_gw:
            gw = _mm(gqt, xqt, sg, sx, out_f32=True).to(ctx.w_dtype)   # [N, M] x [K, M]^T
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = gy.sum(0, dtype=torch.float32)
        return gx, gw, gb, None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           scaling: Optional[LinearScaling] = None) -> torch.Tensor:
    """fp8 ``F.linear`` over any leading dimensions.  ``scaling=None`` scales every tensor by its own maximum (two
    passes per tensor); a :class:`LinearScaling` kept by the caller switches to delayed scaling (one pass).  Feature
    counts and the token count must be multiples of 16, otherwise this is ``F.linear``."""
    k, n = weight.shape[1], weight.shape[0]
    m = x.numel() // max(k, 1)
    if k % 16 or n % 16 or m % 16:
        return torch.nn.functional.linear(x, weight, bias)
    x2d = x.reshape(-1, k)
    if scaling is not None and not (torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad or (bias is not None and bias.requires_grad))):
        # nothing to differentiate: quantise the activation only, the weight's bytes are kept between calls
        x16 = x2d if x2d.dtype in (torch.bfloat16, torch.float16) else x2d.to(torch.bfloat16)
        xq, _, sx = quantize_with(x16, scaling.role("x"))
        wq, sw = scaling.frozen_weight(weight)
        y = _as(_mm(xq, wq, sx, sw, bias=bias), _result_dtype(x))
    else:
        y = _Fp8Linear.apply(x2d, weight, bias, scaling)
    return y.reshape(*x.shape[:-1], n)
