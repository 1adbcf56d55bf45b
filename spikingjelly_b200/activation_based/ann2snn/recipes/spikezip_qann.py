"""SpikeZIP-TF: a quantised ANN (QANN) becomes a spiking network whose time-summed output equals the QANN's output
(You et al., "SpikeZIP-TF: Conversion is All You Need for Transformer-based SNN").

Every activation quantiser of the QANN (a module with a step ``s``, integer limits ``neg_min .. pos_max`` and a
``sym`` flag) becomes a ternary integrate-and-fire neuron (:class:`~...neuron.STBIFNeuron`) that emits ``+s``, ``-s`` or 0
and whose running count stays inside the quantiser's limits; all other operators become temporal-difference operators
that turn the accumulated input into the increment of the accumulated output:

* linear / convolution: linear in the increment; the bias is paid out in ``bias_steps`` equal parts (default: the
  quantisation level), which keeps the neurons behind it from overshooting in the first step;
* embedding: the looked-up vector at the first step, zero afterwards;
* layer norm, softmax, GELU: ``f(sum so far) - f(sum before)``;
* quantised self-attention (any module that exposes ``query / key / value`` or a packed ``qkv`` projection together with
  ``*_quan`` quantisers, the shapes the reference handles for RoBERTa and ViT): the products of two spike trains use
  ``A_t B_t`` increments ``A_sum B_t + A_t B_sum - A_t B_t``, so only increments are multiplied by accumulated values.

Module recipe (no tracing): ``ModuleConverter(recipe=SpikeZIPTFQANNRecipe(time_steps=T)).convert(qann)``; run the result for
``T`` steps with the input at the first step and zeros afterwards (or any split of the input over time) and add the outputs.
Parity: ``spikingjelly/activation_based/ann2snn/recipes/spikezip_qann.py:38-914`` (model-family specific forward patches of
the reference are replaced by one attribute-driven attention wrapper).
"""
from __future__ import annotations

import copy
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import base
from ...neuron.conversion import STBIFNeuron
from ..operators import TDGELU, TDLayerNorm, TDSoftmax
from .base import ModuleConversionRecipe

__all__ = ["SpikeZIPTFQANNRecipe", "SpikeZIPLinear", "SpikeZIPConv2d", "SpikeZIPEmbedding", "SpikeZIPLayerNorm",
           "SpikeZIPSoftmax", "SpikeZIPSelfAttention", "is_quantizer"]


def is_quantizer(module: nn.Module) -> bool:
    return all(hasattr(module, name) for name in ("s", "sym", "pos_max", "neg_min"))


def _level_of(quantizer: nn.Module) -> int:
    if hasattr(quantizer, "level"):
        return int(quantizer.level)
    return int(float(quantizer.pos_max) - float(quantizer.neg_min) + 1)


def _matmul_delta(a, b, a_sum, b_sum, transpose_b: bool = False):
    """Increment of ``A_sum @ B_sum`` when the sums (which already include this step) grew by ``a`` and ``b``."""
    if transpose_b:
        b, b_sum = b.transpose(-1, -2), b_sum.transpose(-1, -2)
    return a_sum @ b + a @ b_sum - a @ b


class _StepwiseModule(base.MemoryModule):
    """Single-step logic in ``step``; multi-step mode loops over the leading axis."""

    def __init__(self, step_mode: str = "s"):
        super().__init__()
        self.step_mode = step_mode

    def step(self, *xs):
        raise NotImplementedError

    def forward(self, *xs):
        if self.step_mode == "s":
            return self.step(*xs)
        return torch.stack([self.step(*(x[t] for x in xs)) for t in range(xs[0].shape[0])])


class _BiasInParts(_StepwiseModule):
    """Affine operator whose bias is released in ``bias_steps`` equal parts, starting when the first non-zero input arrives."""

    def __init__(self, bias: Optional[torch.Tensor], level: int, bias_steps: Optional[int], step_mode: str):
        super().__init__(step_mode)
        self.level = int(level)
        self.bias_steps = self.level if bias_steps is None else int(bias_steps)
        if self.bias_steps <= 0:
            raise ValueError("bias_steps must be positive.")
        if bias is None:
            self.register_parameter("spikezip_bias", None)
        else:
            self.spikezip_bias = nn.Parameter(bias.detach().clone())
        self.register_memory("realize_time", self.bias_steps)
        self.register_memory("is_work", False)

    def _bias_part(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        if not self.is_work and bool((x != 0).any()):
            self.is_work = True
        if self.spikezip_bias is None or not self.is_work or self.realize_time <= 0:
            return None
        self.realize_time = self.realize_time - 1
        return self.spikezip_bias / self.bias_steps


class SpikeZIPLinear(_BiasInParts):
    def __init__(self, linear: nn.Linear, level: int, bias_steps: Optional[int] = None, step_mode: str = "s"):
        super().__init__(linear.bias, level, bias_steps, step_mode)
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.weight = nn.Parameter(linear.weight.detach().clone())

    def step(self, x):
        b = self._bias_part(x)
        return F.linear(x, self.weight, b)


class SpikeZIPConv2d(_BiasInParts):
    def __init__(self, conv: nn.Conv2d, level: int, bias_steps: Optional[int] = None, step_mode: str = "s"):
        super().__init__(conv.bias, level, bias_steps, step_mode)
        self.conv = copy.deepcopy(conv)
        self.conv.bias = None

    def step(self, x):
        b = self._bias_part(x)
        y = self.conv(x)
        return y if b is None else y + b.view(1, -1, 1, 1)


class SpikeZIPEmbedding(_StepwiseModule):
    """Token ids are not a quantity that can be split over time: the embedding is emitted once, then zeros."""

    def __init__(self, embedding: nn.Embedding, step_mode: str = "s"):
        super().__init__(step_mode)
        self.embedding = copy.deepcopy(embedding)
        self.register_memory("emitted", False)

    def step(self, ids):
        y = self.embedding(ids)
        if self.emitted:
            return torch.zeros_like(y)
        self.emitted = True
        return y


class SpikeZIPLayerNorm(TDLayerNorm):
    def __init__(self, source: nn.LayerNorm, step_mode: str = "s"):
        super().__init__(source.normalized_shape, eps=source.eps, elementwise_affine=source.elementwise_affine,
                         bias=source.bias is not None, step_mode=step_mode, device=source.weight.device if source.elementwise_affine else None)
        self.norm.load_state_dict(source.state_dict())


class SpikeZIPSoftmax(TDSoftmax):
    def __init__(self, dim: int = -1, step_mode: str = "s"):
        super().__init__(dim, step_mode=step_mode)


def _neuron(quantizer: Optional[nn.Module]):
    return nn.Identity() if quantizer is None or not is_quantizer(quantizer) else STBIFNeuron.from_quantizer(quantizer)


class SpikeZIPSelfAttention(_StepwiseModule):
    """Quantised multi-head self-attention as spikes.  Source attributes (first match wins):

    projections   ``query, key, value`` (three linears)  or  ``qkv`` (one packed linear, columns ordered q | k | v)
    quantisers    ``query_quan | quan_q``, ``key_quan | quan_k``, ``value_quan | quan_v`` behind the projections,
                  ``attn_quan`` behind the softmax, ``after_attn_quan`` behind the context product
    head count    ``num_attention_heads | num_heads``;  scale ``scale`` or ``head_dim ** -0.5``
    output        optional ``proj`` (linear) and ``proj_quan | quan_proj``
    """

    def __init__(self, source: nn.Module, level: int, step_mode: str = "s"):
        super().__init__(step_mode)
        pick = lambda *names: next((getattr(source, n) for n in names if getattr(source, n, None) is not None), None)  # noqa: E731
        self.level = int(level)
        self.num_heads = int(pick("num_attention_heads", "num_heads"))
        self.packed = getattr(source, "qkv", None) is not None
        if self.packed:
            self.qkv = SpikeZIPLinear(source.qkv, level)
            dim = source.qkv.out_features // 3
        else:
            self.query, self.key, self.value = (SpikeZIPLinear(getattr(source, n), level) for n in ("query", "key", "value"))
            dim = source.query.out_features
        self.head_dim = dim // self.num_heads
        scale = getattr(source, "scale", None)
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        self.query_if, self.key_if, self.value_if = _neuron(pick("query_quan", "quan_q")), _neuron(pick("key_quan", "quan_k")), _neuron(pick("value_quan", "quan_v"))
        self.softmax = SpikeZIPSoftmax(-1)
        self.attn_if = _neuron(pick("attn_quan"))
        self.after_attn_if = _neuron(pick("after_attn_quan"))
        proj = pick("proj")
        self.proj = SpikeZIPLinear(proj, level) if isinstance(proj, nn.Linear) else None
        self.proj_if = _neuron(pick("proj_quan", "quan_proj")) if self.proj is not None else None
        for name in ("q_sum", "k_sum", "v_sum", "p_sum"):
            self.register_memory(name, None)

    def _heads(self, x):                                  # [B, L, C] -> [B, H, L, D]
        b, l, _ = x.shape
        return x.view(b, l, self.num_heads, self.head_dim).transpose(1, 2)

    @staticmethod
    def _acc(total, x):
        return x if total is None or not torch.is_tensor(total) or total.shape != x.shape else total + x

    def step(self, x):
        if self.packed:
            q, k, v = self.qkv(x).chunk(3, dim=-1)
        else:
            q, k, v = self.query(x), self.key(x), self.value(x)
        q, k, v = self._heads(self.query_if(q)), self._heads(self.key_if(k)), self._heads(self.value_if(v))
        self.q_sum, self.k_sum, self.v_sum = self._acc(self.q_sum, q), self._acc(self.k_sum, k), self._acc(self.v_sum, v)
        scores = _matmul_delta(q, k, self.q_sum, self.k_sum, transpose_b=True) * self.scale
        p = self.attn_if(self.softmax(scores))
        self.p_sum = self._acc(self.p_sum, p)
        ctx = self.after_attn_if(_matmul_delta(p, v, self.p_sum, self.v_sum))
        b, _, l, _ = ctx.shape
        out = ctx.transpose(1, 2).reshape(b, l, self.num_heads * self.head_dim)
        if self.proj is not None:
            out = self.proj_if(self.proj(out))
        return out


def _is_qattention(module: nn.Module) -> bool:
    has_proj = getattr(module, "qkv", None) is not None or all(getattr(module, n, None) is not None for n in ("query", "key", "value"))
    has_quan = any(getattr(module, n, None) is not None for n in ("query_quan", "quan_q"))
    has_heads = any(hasattr(module, n) for n in ("num_attention_heads", "num_heads"))
    return has_proj and has_quan and has_heads


class SpikeZIPTFQANNRecipe(ModuleConversionRecipe):
    """``time_steps``: the number of steps the converted model is meant to run (stored on it as ``time_steps``; also the
    fallback quantisation level when the QANN has no quantiser).  ``model_family`` (``"roberta"``, ``"vit"`` or
    ``"generic"``) is recorded on the result; the conversion itself is driven by module attributes, not by the family."""

    def __init__(self, time_steps: int = 200, model_family: str = "roberta") -> None:
        self.time_steps, self.model_family = time_steps, model_family

    def validate(self, converter) -> None:
        if not isinstance(self.time_steps, int) or isinstance(self.time_steps, bool) or self.time_steps <= 0:
            raise ValueError("time_steps must be a positive integer.")
        if self.model_family not in ("roberta", "vit", "generic"):
            raise ValueError("SpikeZIPTFQANNRecipe supports model_family='roberta', 'vit' or 'generic'.")

    def _level_from_model(self, model: nn.Module) -> int:
        for m in model.modules():
            if is_quantizer(m):
                return _level_of(m)
        return self.time_steps

    @staticmethod
    def _attention_level(module: nn.Module) -> int:
        for name in ("query_quan", "key_quan", "value_quan", "quan_q", "quan_k", "quan_v"):
            q = getattr(module, name, None)
            if q is not None and (hasattr(q, "level") or is_quantizer(q)):
                return _level_of(q)
        raise ValueError("SpikeZIP QANN attention must expose quantizer level.")

    def _replace(self, model: nn.Module, level: int) -> None:
        for name, child in list(model.named_children()):
            new = None
            if _is_qattention(child):
                new = SpikeZIPSelfAttention(child, self._attention_level(child))
            elif isinstance(child, nn.Embedding):
                new = SpikeZIPEmbedding(child)
            elif isinstance(child, nn.Conv2d):
                new = SpikeZIPConv2d(child, level)
            elif isinstance(child, nn.Linear):
                new = SpikeZIPLinear(child, level)
            elif isinstance(child, nn.LayerNorm):
                new = SpikeZIPLayerNorm(child)
            elif isinstance(child, nn.Softmax):
                new = SpikeZIPSoftmax(child.dim if child.dim is not None else -1)
            elif isinstance(child, nn.GELU):
                new = TDGELU(child.approximate, step_mode="s")
            elif is_quantizer(child):
                new = STBIFNeuron.from_quantizer(child)
            elif isinstance(child, nn.ReLU):
                new = nn.Identity()          # the unsigned quantiser behind a ReLU already clips at zero
            if new is None:
                self._replace(child, level)
            else:
                if isinstance(new, base.StepModule) and hasattr(new, "step_mode") and not isinstance(new, STBIFNeuron):
                    new.step_mode = "s"
                setattr(model, name, new)

    def convert_module(self, converter, ann: nn.Module) -> nn.Module:
        model = copy.deepcopy(ann).eval()
        self._replace(model, self._level_from_model(model))
        model.ann2snn_recipe = "spikezip_tf_qann"
        model.time_steps = self.time_steps
        model.model_family = self.model_family
        return model
