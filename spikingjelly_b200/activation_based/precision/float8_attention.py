"""Adapter with the interface of a ``[B, H, L, D]`` dot-product-attention module.  The attention itself
runs through ``F.scaled_dot_product_attention`` under the surrounding autocast (bf16): attention
probabilities do not survive fp8 quantisation well, so only the projections around it are fp8.
Parity: ``spikingjelly/activation_based/precision/float8_attention.py:1-175`` (the reference routes
this to Transformer Engine's ``DotProductAttention``)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["TransformerEngineDotProductAttentionAdapter"]


class TransformerEngineDotProductAttentionAdapter(nn.Module):
    def __init__(self, num_heads: int, head_dim: int, attention_dropout: float = 0.0, qkv_format: str = "bhsd",
                 attn_mask_type: str = "no_mask", softmax_scale: Optional[float] = None):
        super().__init__()
        if qkv_format not in ("bhsd", "bshd", "sbhd"):
            raise ValueError(f"Unsupported qkv_format {qkv_format!r}.")
        if attn_mask_type not in ("no_mask", "causal", "arbitrary"):
            raise ValueError(f"Unsupported attn_mask_type {attn_mask_type!r}.")
        self.num_heads, self.head_dim = num_heads, head_dim
        self.attention_dropout, self.qkv_format, self.attn_mask_type = attention_dropout, qkv_format, attn_mask_type
        self.softmax_scale = softmax_scale

    def _to_bhsd(self, t):
        return {"bhsd": lambda x: x, "bshd": lambda x: x.transpose(1, 2), "sbhd": lambda x: x.permute(1, 2, 0, 3)}[self.qkv_format](t)

    def _from_bhsd(self, t):
        return {"bhsd": lambda x: x, "bshd": lambda x: x.transpose(1, 2), "sbhd": lambda x: x.permute(2, 0, 1, 3)}[self.qkv_format](t)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, attention_mask: Optional[torch.Tensor] = None):
        q, k, v = (self._to_bhsd(t) for t in (q, k, v))
        if q.shape[1] != self.num_heads or q.shape[-1] != self.head_dim:
            raise ValueError(f"expected {self.num_heads} heads of size {self.head_dim}, got {tuple(q.shape)}")
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=attention_mask if self.attn_mask_type == "arbitrary" else None,
                                             dropout_p=self.attention_dropout if self.training else 0.0,
                                             is_causal=self.attn_mask_type == "causal", scale=self.softmax_scale)
        return self._from_bhsd(out)
