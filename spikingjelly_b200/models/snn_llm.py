"""Spike-driven decoder-only language model ("SNN-LLM"): 24 layers, d = 2048, 16 heads, FFN 5504, RMSNorm,
rotary position embedding, vocabulary 32000, LIF neurons (tau = 2) simulated for T = 4 steps.

The reference tree has no trainable model of this shape (it has an inference-only Qwen2 conversion and runners for
an external SpikeGPT tree); this definition is assembled from the same public parts a reference user would use —
``layer.Linear``, ``neuron.LIFNode`` in multi-step mode, plain PyTorch attention — so that the module graph is
expressible on both frameworks.  Every matrix multiplication consumes spikes:

    s   = LIF(RMSNorm(h))                       h: real-valued residual stream [T, B, S, d]
    q,k,v = Linear(s) ; a = causal SDPA(rope(q), rope(k), v) ; h += Linear(LIF(a))
    s2  = LIF(RMSNorm(h))       ; h += Linear(LIF(Linear(s2)))

Tensor parallelism (:func:`parallelize_snn_llm`): heads and FFN columns are sharded (column-parallel QKV / up,
row-parallel O / down).  The fused path (``parallel/fused_tp.py``) additionally shards the residual stream by
tokens, all-gathers the 1-bit spikes inside the column-parallel GEMM and reduce-scatters inside the row-parallel
GEMM's epilogue.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..activation_based import functional, layer, neuron, surrogate
from ..ops import rope as rope_ops

__all__ = ["SNNLLMConfig", "RMSNorm", "RotaryEmbedding", "SpikingCausalSelfAttention", "SpikingFFN", "SNNLLMBlock",
           "SNNLLM", "snn_llm_1b", "snn_llm_tiny", "parallelize_snn_llm"]


@dataclass
class SNNLLMConfig:
    vocab_size: int = 32000
    d_model: int = 2048
    n_layers: int = 24
    n_heads: int = 16
    d_ffn: int = 5504
    T: int = 4
    tau: float = 2.0
    max_seq_len: int = 2048
    rope_theta: float = 10000.0
    rms_eps: float = 1e-6
    backend: str = "torch"
    tie_embeddings: bool = False

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """fp32 statistics; the result is returned in the autocast compute dtype when autocast is on (the neuron that
        follows then reads and writes 16-bit tensors), else in ``x``'s dtype."""
        out_dtype = x.dtype
        if x.is_cuda and torch.is_autocast_enabled("cuda"):
            out_dtype = torch.get_autocast_dtype("cuda")
        if x.is_cuda:
            with torch.autocast("cuda", enabled=False):
                return F.rms_norm(x.float() if x.dtype != torch.float32 else x, (x.shape[-1],), self.weight.float(), self.eps).to(out_dtype)
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (y * self.weight.float()).to(out_dtype)


class RotaryEmbedding(nn.Module):
    """Rotates pairs ``(x[..., i], x[..., i + D/2])`` by ``pos * theta^(-2i/D)`` (the half-split convention)."""

    def __init__(self, head_dim: int, max_seq_len: int, theta: float = 10000.0):
        super().__init__()
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
        ang = torch.outer(torch.arange(max_seq_len).float(), inv)
        self.register_buffer("cos", torch.cat([ang.cos(), ang.cos()], -1), persistent=False)
        self.register_buffer("sin", torch.cat([ang.sin(), ang.sin()], -1), persistent=False)

    def forward(self, x: torch.Tensor, offset: int = 0) -> torch.Tensor:
        S = x.shape[-2]                                                # x: [..., heads, S, D]
        cos, sin = self.cos[offset:offset + S].to(x.dtype), self.sin[offset:offset + S].to(x.dtype)
        half = x.shape[-1] // 2
        rot = torch.cat([-x[..., half:], x[..., :half]], -1)
        return x * cos + rot * sin


def _lif(cfg: SNNLLMConfig) -> neuron.LIFNode:
    return neuron.LIFNode(tau=cfg.tau, detach_reset=True, surrogate_function=surrogate.ATan(), step_mode="m", backend=cfg.backend)


class SpikingCausalSelfAttention(nn.Module):
    """Spikes in, real-valued increment of the residual stream out.  ``n_local_heads`` shrinks under TP."""

    def __init__(self, cfg: SNNLLMConfig):
        super().__init__()
        self.cfg = cfg
        self.n_local_heads = cfg.n_heads
        self.qkv = layer.Linear(cfg.d_model, 3 * cfg.d_model, bias=False, step_mode="m")
        self.attn_lif = _lif(cfg)
        self.proj = layer.Linear(cfg.d_model, cfg.d_model, bias=False, step_mode="m")
        self.rope = RotaryEmbedding(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta)

    def forward(self, s: torch.Tensor) -> torch.Tensor:
        T, B, S, _ = s.shape
        H, D = self.n_local_heads, self.cfg.head_dim
        qkv = self.qkv(s).reshape(T * B, S, H, 3, D)                     # head-major so that TP shards whole heads
        if rope_ops.supports(qkv, D):
            # one kernel: rotate q and k, split; the results are [T*B, S, H, D] in memory, which is also the order the
            # attention output comes back in, so neither side needs a layout copy
            q, k, v = (t.transpose(1, 2) for t in rope_ops.rope_qkv(qkv, self.rope.cos, self.rope.sin))
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        else:
            q, k, v = (qkv[:, :, :, i].transpose(1, 2) for i in range(3))    # [T*B, H, S, D]
            a = F.scaled_dot_product_attention(self.rope(q), self.rope(k), v, is_causal=True)
        a = a.transpose(1, 2).reshape(T, B, S, H * D)
        return self.proj(self.attn_lif(a))


class SpikingFFN(nn.Module):
    def __init__(self, cfg: SNNLLMConfig):
        super().__init__()
        self.up = layer.Linear(cfg.d_model, cfg.d_ffn, bias=False, step_mode="m")
        self.lif = _lif(cfg)
        self.down = layer.Linear(cfg.d_ffn, cfg.d_model, bias=False, step_mode="m")

    def forward(self, s: torch.Tensor) -> torch.Tensor:
        return self.down(self.lif(self.up(s)))


class SNNLLMBlock(nn.Module):
    def __init__(self, cfg: SNNLLMConfig):
        super().__init__()
        self.norm1, self.lif1, self.attn = RMSNorm(cfg.d_model, cfg.rms_eps), _lif(cfg), SpikingCausalSelfAttention(cfg)
        self.norm2, self.lif2, self.ffn = RMSNorm(cfg.d_model, cfg.rms_eps), _lif(cfg), SpikingFFN(cfg)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        h = h + self.attn(self.lif1(self.norm1(h)))
        return h + self.ffn(self.lif2(self.norm2(h)))


class SNNLLM(nn.Module):
    """``forward(tokens[B, S]) -> logits[B, S, vocab]``; with ``labels`` also the mean next-token cross entropy.
    The token embedding is presented at each of the ``T`` steps (direct encoding); logits read the mean over ``T``."""

    def __init__(self, cfg: SNNLLMConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.blocks = nn.ModuleList(SNNLLMBlock(cfg) for _ in range(cfg.n_layers))
        self.norm_f = RMSNorm(cfg.d_model, cfg.rms_eps)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.embed.weight
        self.apply(self._init)
        for name, p in self.named_parameters():
            if name.endswith("proj.weight") or name.endswith("down.weight"):
                nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * cfg.n_layers))

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def flops_per_token(self, seq_len: int) -> float:
        """Forward multiply-accumulate FLOPs (x2) per token and time step, attention included."""
        c = self.cfg
        per_layer = 2 * (4 * c.d_model * c.d_model + 2 * c.d_model * c.d_ffn) + 4 * seq_len * c.d_model / 2
        return c.T * c.n_layers * per_layer + 2 * c.d_model * c.vocab_size

    def forward(self, tokens: torch.Tensor, labels: Optional[torch.Tensor] = None):
        functional.reset_net(self)
        x = self.embed(tokens)                                            # [B, S, d]
        h = x.unsqueeze(0).expand(self.cfg.T, *x.shape)
        for blk in self.blocks:
            h = blk(h)
        logits = self.lm_head(self.norm_f(h.mean(0)))
        if labels is None:
            return logits
        loss = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), labels[:, 1:].reshape(-1))
        return logits, loss


def snn_llm_1b(**overrides) -> SNNLLM:
    """The benchmark shape: 24 layers, d 2048, 16 heads, FFN 5504, vocabulary 32000, T = 4 (about 1.3 B parameters)."""
    return SNNLLM(SNNLLMConfig(**overrides))


def snn_llm_tiny(**overrides) -> SNNLLM:
    cfg = dict(vocab_size=256, d_model=64, n_layers=2, n_heads=4, d_ffn=128, T=2, max_seq_len=64)
    cfg.update(overrides)
    return SNNLLM(SNNLLMConfig(**cfg))


def parallelize_snn_llm(model: SNNLLM, group=None) -> SNNLLM:
    """Megatron-style tensor parallelism over ``group``: QKV and up are split by output features (whole heads / FFN
    columns), O and down by input features with an all-reduce of their outputs; norms, LIFs of the residual stream,
    embedding and LM head stay replicated.  Gradients of replicated parameters are identical on all ranks."""
    import torch.distributed as dist
    from ..parallel import tensor_parallel as tp
    ws = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if ws == 1:
        return model
    cfg = model.cfg
    if cfg.n_heads % ws or cfg.d_ffn % ws:
        raise ValueError(f"n_heads ({cfg.n_heads}) and d_ffn ({cfg.d_ffn}) must be divisible by the group size {ws}")
    for blk in model.blocks:
        a = blk.attn
        a.n_local_heads = cfg.n_heads // ws
        a.qkv = tp.ColwiseParallelLinear(a.qkv, group)          # rows of W are head-major: a contiguous slice = whole heads
        a.proj = tp.RowwiseParallelLinear(a.proj, group)
        blk.ffn.up = tp.ColwiseParallelLinear(blk.ffn.up, group)
        blk.ffn.down = tp.RowwiseParallelLinear(blk.ffn.down, group)
    return model
