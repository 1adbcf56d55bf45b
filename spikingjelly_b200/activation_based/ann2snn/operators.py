"""Temporal-difference (TD) operators: exact spike-domain equivalents of ANN operators.

A TD operator keeps the running sums of its inputs and of the ANN operator's output; at step ``t``
it emits ``f(sum_{s<=t} x_s) - f(sum_{s<t} x_s)``.  The outputs therefore telescope:
``sum_t y_t == f(sum_t x_t)`` for *any* ``f`` — softmax, layer norm, GELU, attention, products of two
sequences — which is what makes transformer blocks convertible without approximation.  Linear
operators need no state beyond the bias bookkeeping (``f(a + b) - f(a) = W b``), but keep the same
interface.

Multi-step mode evaluates ``f`` once on the cumulative sum over the whole sequence (time folded into
the batch) and differences along time: one kernel launch per operator instead of ``T``.

Parity: ``spikingjelly/activation_based/ann2snn/operators.py:12-2985``.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import base

__all__ = ["TDModule", "TDSoftmax", "TDLayerNorm", "TDRMSNorm", "TDGELU", "TDSiLU", "TDLinear", "TDConv2d", "SNNMatrixOperator",
           "SNNElementWiseProduct", "TDScaledDotProductAttention", "TDMultiheadAttention"]


def _temporal_difference(y_cum: torch.Tensor, previous: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = torch.empty_like(y_cum)
    y[0] = y_cum[0] if previous is None else y_cum[0] - previous
    y[1:] = y_cum[1:] - y_cum[:-1]
    return y


def _same_meta(a, b) -> bool:
    return isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and a.shape == b.shape and a.device == b.device and a.dtype == b.dtype


class TDModule(base.MemoryModule):
    """Base class: subclasses implement ``ann_forward(*accumulated_inputs)``.  ``time_batched = True``
    promises that ``ann_forward`` treats dimension 0 as a batch dimension, so a whole sequence can be
    evaluated in one call with time folded into the batch."""
    time_batched = True

    def __init__(self, step_mode: str = "m") -> None:
        super().__init__()
        self.register_memory("x_cum", None)
        self.register_memory("y_cum", None)
        self.step_mode = step_mode

    def ann_forward(self, *args, **kwargs):
        raise NotImplementedError

    # -- single step ------------------------------------------------------------------------
    def single_step_forward(self, *inputs, **kwargs):
        prev = self.x_cum if isinstance(self.x_cum, tuple) else (self.x_cum,)
        if len(prev) != len(inputs) or not all(_same_meta(p, c) for p, c in zip(prev, inputs)):
            prev, self.y_cum = (None,) * len(inputs), None
        acc = tuple(c if p is None else p + c for p, c in zip(prev, inputs))
        self.x_cum = acc[0] if len(acc) == 1 else acc
        y_cum = self.ann_forward(*acc, **kwargs)
        y = y_cum - self.y_cum if _same_meta(self.y_cum, y_cum) else y_cum
        self.y_cum = y_cum
        return y

    # -- whole sequence ---------------------------------------------------------------------
    def _sequence_ann(self, *cum_seqs, **kwargs):
        if self.time_batched:
            T = cum_seqs[0].shape[0]
            y = self.ann_forward(*(c.flatten(0, 1) for c in cum_seqs), **kwargs)
            return y.reshape(T, -1, *y.shape[1:])
        return torch.stack([self.ann_forward(*(c[t] for c in cum_seqs), **kwargs) for t in range(cum_seqs[0].shape[0])])

    def multi_step_forward(self, *input_seqs, **kwargs):
        for x in input_seqs:
            if x.dim() < 2:
                raise ValueError(f"{type(self).__name__} expects an input sequence with shape [T, ...] and at least 2 dimensions, "
                                 f"but got shape {tuple(x.shape)}.")
            if x.shape[0] == 0:
                raise ValueError(f"{type(self).__name__} expects a non-empty time dimension, but got shape {tuple(x.shape)}.")
        cums = tuple(x.cumsum(dim=0) for x in input_seqs)
        prev = self.x_cum if isinstance(self.x_cum, tuple) else (self.x_cum,)
        if len(prev) == len(cums) and all(_same_meta(p, c[0]) for p, c in zip(prev, cums)):
            cums = tuple(p + c for p, c in zip(prev, cums))
            y_prev = self.y_cum
        else:
            y_prev = None
        y_cum_seq = self._sequence_ann(*cums, **kwargs)
        y = _temporal_difference(y_cum_seq, y_prev if _same_meta(y_prev, y_cum_seq[0]) else None)
        finals = tuple(c[-1].clone() for c in cums)
        self.x_cum = finals[0] if len(finals) == 1 else finals
        self.y_cum = y_cum_seq[-1].clone()
        return y

    def forward(self, *inputs, **kwargs):
        if self.step_mode == "s":
            return self.single_step_forward(*inputs, **kwargs)
        if self.step_mode == "m":
            return self.multi_step_forward(*inputs, **kwargs)
        raise ValueError(self.step_mode)

    def reset_parameters(self) -> None:
        """Re-initialises the wrapped ANN operator(s) the way their own ``reset_parameters`` does."""
        for m in self.children():
            if hasattr(m, "reset_parameters"):
                m.reset_parameters()


class TDSoftmax(TDModule):
    def __init__(self, dim: int = -1, step_mode: str = "m") -> None:
        super().__init__(step_mode)
        self.dim = dim

    def ann_forward(self, x):
        if self.dim >= 0 and self.time_batched and self.step_mode == "m":
            pass
        return torch.softmax(x, dim=self.dim)

    def extra_repr(self):
        return f"dim={self.dim}, step_mode={self.step_mode}"


class TDLayerNorm(TDModule):
    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True, bias: bool = True, device=None, dtype=None,
                 step_mode: str = "m") -> None:
        super().__init__(step_mode)
        self.norm = nn.LayerNorm(normalized_shape, eps=eps, elementwise_affine=elementwise_affine, bias=bias, device=device, dtype=dtype)

    @classmethod
    def from_ann(cls, m: nn.LayerNorm, step_mode: str = "m"):
        new = cls(m.normalized_shape, m.eps, m.elementwise_affine, m.bias is not None, step_mode=step_mode)
        new.norm = m
        return new

    @property
    def weight(self):
        return self.norm.weight

    @property
    def bias(self):
        return self.norm.bias

    def ann_forward(self, x):
        return self.norm(x)


class TDRMSNorm(TDModule):
    def __init__(self, normalized_shape, eps: Optional[float] = None, elementwise_affine: bool = True, device=None, dtype=None,
                 step_mode: str = "m") -> None:
        super().__init__(step_mode)
        self.normalized_shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(self.normalized_shape, device=device, dtype=dtype)) if elementwise_affine else None

    @classmethod
    def from_ann(cls, m, step_mode: str = "m"):
        new = cls(m.normalized_shape, getattr(m, "eps", None), getattr(m, "weight", None) is not None, step_mode=step_mode)
        if getattr(m, "weight", None) is not None:
            new.weight = m.weight
        return new

    def ann_forward(self, x):
        return F.rms_norm(x, self.normalized_shape, self.weight, self.eps)

    def reset_parameters(self) -> None:
        if self.weight is not None:
            nn.init.ones_(self.weight)


class TDGELU(TDModule):
    def __init__(self, approximate: str = "none", step_mode: str = "m") -> None:
        super().__init__(step_mode)
        self.approximate = approximate

    def ann_forward(self, x):
        return F.gelu(x, approximate=self.approximate)


class TDSiLU(TDModule):
    def ann_forward(self, x):
        return F.silu(x)


class TDLinear(TDModule):
    """``y_t = W x_t`` (+ ``b`` on the first step only: the bias belongs to the accumulated output once)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None, step_mode: str = "m") -> None:
        super().__init__(step_mode)
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=dtype)) if bias else None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.in_features)
            nn.init.uniform_(self.bias, -bound, bound)

    @classmethod
    def from_ann(cls, m: nn.Linear, step_mode: str = "m"):
        new = cls.__new__(cls)
        TDModule.__init__(new, step_mode)
        new.in_features, new.out_features, new.weight, new.bias = m.in_features, m.out_features, m.weight, m.bias
        return new

    def ann_forward(self, x):
        return F.linear(x, self.weight, self.bias)

    def single_step_forward(self, x):
        first = not isinstance(self.y_cum, torch.Tensor)
        y = F.linear(x, self.weight, self.bias if first else None)
        self.x_cum = x if first or not _same_meta(self.x_cum, x) else self.x_cum + x
        self.y_cum = y if first else self.y_cum + y
        return y

    def multi_step_forward(self, x_seq):
        if x_seq.dim() < 2 or x_seq.shape[0] == 0:
            raise ValueError(f"TDLinear expects a non-empty sequence [T, ...], but got shape {tuple(x_seq.shape)}.")
        first = not isinstance(self.y_cum, torch.Tensor)
        y = F.linear(x_seq, self.weight)
        if self.bias is not None and first:
            y[0] = y[0] + self.bias
        total = x_seq.sum(0)
        self.x_cum = total if first or not _same_meta(self.x_cum, total) else self.x_cum + total
        ysum = y.sum(0)
        self.y_cum = ysum if first else self.y_cum + ysum
        return y

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, step_mode={self.step_mode}"


class TDConv2d(TDModule):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode="zeros", device=None, dtype=None, step_mode: str = "m") -> None:
        super().__init__(step_mode)
        self.conv = nn.Conv2d(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias, padding_mode,
                              device=device, dtype=dtype)

    @classmethod
    def from_ann(cls, m: nn.Conv2d, step_mode: str = "m"):
        new = cls.__new__(cls)
        TDModule.__init__(new, step_mode)
        new.conv = m
        return new

    @property
    def weight(self):
        return self.conv.weight

    @property
    def bias(self):
        return self.conv.bias

    def ann_forward(self, x):
        return self.conv(x)


class SNNMatrixOperator(TDModule):
    """``A @ B`` of two activation sequences (both accumulate): ``y_t = A_cum B_cum - (previous)``.
    ``transpose_b`` contracts with ``B^T`` (attention scores)."""

    def __init__(self, step_mode: str = "m", transpose_b: bool = False, scale: Optional[float] = None) -> None:
        super().__init__(step_mode)
        self.transpose_b, self.scale = transpose_b, scale

    def ann_forward(self, a, b):
        y = torch.matmul(a, b.transpose(-1, -2) if self.transpose_b else b)
        return y if self.scale is None else y * self.scale


class SNNElementWiseProduct(TDModule):
    def ann_forward(self, a, b):
        return a * b


class TDScaledDotProductAttention(TDModule):
    """``softmax(Q K^T / sqrt(d) + mask) V`` on accumulated Q, K, V (``[..., L, E]``)."""

    def __init__(self, is_causal: bool = False, scale: Optional[float] = None, step_mode: str = "m", dropout_p: float = 0.0) -> None:
        super().__init__(step_mode)
        if dropout_p != 0.0:
            raise ValueError("TDScaledDotProductAttention is deterministic: dropout_p must be 0.")
        self.is_causal, self.scale = is_causal, scale
        self.attn_mask = None

    def ann_forward(self, query, key, value, attn_mask: Optional[torch.Tensor] = None):
        q, k, v = query, key, value
        mask = self.attn_mask if attn_mask is None else attn_mask
        if mask is not None and mask.dim() == q.dim() and mask.shape[0] not in (1, q.shape[0]) and q.shape[0] % mask.shape[0] == 0:
            # a whole sequence is evaluated with time folded into the batch (time-major): the per-sample mask repeats
            mask = mask.repeat(q.shape[0] // mask.shape[0], *([1] * (mask.dim() - 1)))
        return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, is_causal=self.is_causal and mask is None, scale=self.scale)

    def forward(self, query, key, value, attn_mask: Optional[torch.Tensor] = None):
        self.attn_mask = attn_mask
        try:
            return super().forward(query, key, value)
        finally:
            self.attn_mask = None


class TDMultiheadAttention(TDModule):
    """``nn.MultiheadAttention`` (self- or cross-attention, ``batch_first`` either way) as one TD
    operator: the projections, the attention and the output projection are applied to the
    accumulated query / key / value.  Returns ``(output, None)`` like the ANN module with
    ``need_weights=False``."""
    time_batched = False

    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True, batch_first: bool = True, device=None,
                 dtype=None, step_mode: str = "m") -> None:
        super().__init__(step_mode)
        if dropout != 0.0:
            raise ValueError("TDMultiheadAttention is deterministic: dropout must be 0.")
        self.mha = nn.MultiheadAttention(embed_dim, num_heads, bias=bias, batch_first=batch_first, device=device, dtype=dtype)

    @classmethod
    def from_ann(cls, m: nn.MultiheadAttention, step_mode: str = "m"):
        if m.dropout != 0.0 and m.training:
            raise ValueError("TDMultiheadAttention requires dropout == 0 or eval mode.")
        new = cls.__new__(cls)
        TDModule.__init__(new, step_mode)
        new.mha = m
        return new

    def ann_forward(self, query, key, value, key_padding_mask=None, need_weights: bool = False, attn_mask=None,
                    average_attn_weights: bool = True, is_causal: bool = False):
        if need_weights:
            raise ValueError("TDMultiheadAttention returns no attention weights: need_weights must be False.")
        return self.mha(query, key, value, key_padding_mask=key_padding_mask, need_weights=False, attn_mask=attn_mask, is_causal=is_causal)[0]

    def forward(self, query, key=None, value=None, **kwargs):
        key = query if key is None else key
        value = key if value is None else value
        kwargs.pop("need_weights", None)
        return super().forward(query, key, value, **kwargs), None


def _td_module_from_ann(module: nn.Module, step_mode: str = "m") -> Optional[nn.Module]:
    """The TD operator equivalent to an ANN module, or None when there is none."""
    if isinstance(module, nn.Linear):
        return TDLinear.from_ann(module, step_mode)
    if isinstance(module, nn.Conv2d):
        return TDConv2d.from_ann(module, step_mode)
    if isinstance(module, nn.LayerNorm):
        return TDLayerNorm.from_ann(module, step_mode)
    if hasattr(nn, "RMSNorm") and isinstance(module, nn.RMSNorm):
        return TDRMSNorm.from_ann(module, step_mode)
    if isinstance(module, nn.GELU):
        return TDGELU(getattr(module, "approximate", "none"), step_mode)
    if isinstance(module, nn.SiLU):
        return TDSiLU(step_mode)
    if isinstance(module, nn.Softmax):
        return TDSoftmax(-1 if module.dim is None else module.dim, step_mode)
    if isinstance(module, nn.MultiheadAttention):
        return TDMultiheadAttention.from_ann(module, step_mode)
    return None
