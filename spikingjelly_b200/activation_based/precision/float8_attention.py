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
    def __init__(self, num_attention_heads: int, head_dim: int, attention_dropout: float = 0.0, qkv_format: str = "bhsd",
                 attn_mask_type: str = "no_mask", softmax_scale: Optional[float] = None):
        super().__init__()
        if qkv_format not in ("bhsd", "bshd", "sbhd"):
            raise ValueError(f"Unsupported qkv_format {qkv_format!r}.")
        if attn_mask_type not in ("no_mask", "causal", "arbitrary"):
            raise ValueError(f"Unsupported attn_mask_type {attn_mask_type!r}.")
        self.num_attention_heads, self.head_dim = num_attention_heads, head_dim
        self.attention_dropout, self.qkv_format, self.attn_mask_type = attention_dropout, qkv_format, attn_mask_type
        self.softmax_scale = softmax_scale

    @property
    def num_heads(self) -> int:
        return self.num_attention_heads

    def _to_bhsd(self, t):
        return {"bhsd": lambda x: x, "bshd": lambda x: x.transpose(1, 2), "sbhd": lambda x: x.permute(1, 2, 0, 3)}[self.qkv_format](t)

    def _from_bhsd(self, t):
        return {"bhsd": lambda x: x, "bshd": lambda x: x.transpose(1, 2), "sbhd": lambda x: x.permute(2, 0, 1, 3)}[self.qkv_format](t)

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, attn_mask: Optional[torch.Tensor] = None,
                dropout_p: float = 0.0, is_causal: bool = False, scale: Optional[float] = None, *, attention_mask=None):
        """The arguments of ``F.scaled_dot_product_attention``.  ``attn_mask`` is used when the adapter was built with
        ``attn_mask_type="arbitrary"``; ``is_causal`` or ``attn_mask_type="causal"`` gives the causal mask; ``dropout_p``, when given,
        must agree with the adapter's own (``attention_dropout`` in training, 0 in evaluation)."""
        attn_mask = attention_mask if attn_mask is None else attn_mask
        expected = self.attention_dropout if self.training else 0.0
        if dropout_p != 0.0 and abs(dropout_p - expected) > 1e-12:      # 0.0 (the default) means: the adapter's own setting
            raise ValueError(f"dropout_p={dropout_p} disagrees with the adapter ({expected} in this mode).")
        q, k, v = (self._to_bhsd(t) for t in (query, key, value))
        for name, t in (("query", q), ("key", k), ("value", v)):
            if t.dim() != 4 or t.shape[1] != self.num_attention_heads or t.shape[-1] != self.head_dim:
                raise ValueError(f"{name}: expected {self.num_attention_heads} heads of size {self.head_dim}, got {tuple(t.shape)}")
        causal = is_causal or self.attn_mask_type == "causal"
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask if self.attn_mask_type == "arbitrary" else None, dropout_p=expected,
                                             is_causal=causal, scale=self.softmax_scale if scale is None else scale)
        return self._from_bhsd(out)
