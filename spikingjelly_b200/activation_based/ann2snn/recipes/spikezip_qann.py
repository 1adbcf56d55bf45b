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
import types
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import base
from ...neuron.conversion import STBIFNeuron
from ..operators import TDGELU, TDLayerNorm, TDSoftmax
from .base import ModuleConversionRecipe

__all__ = ["SpikeZIPTFQANNRecipe", "SpikeZIPLinear", "SpikeZIPConv2d", "SpikeZIPEmbedding", "SpikeZIPLayerNorm",
           "SpikeZIPSoftmax", "SpikeZIPSelfAttention", "SpikeZIPRobertaSelfAttention", "SpikeZIPViTSelfAttention", "is_quantizer"]


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


def _matmul_delta_sequence(a_seq, b_seq, a_prev, b_prev, transpose_b: bool = False):
    """``_matmul_delta`` for every step of ``[T, ...]`` sequences in three batched products; ``a_prev`` / ``b_prev`` are
    the sums before the first step (``None`` = zero).  Returns ``(increments, a_sum_last, b_sum_last)``."""
    a_sum, b_sum = a_seq.cumsum(0), b_seq.cumsum(0)
    if a_prev is not None:
        a_sum, b_sum = a_sum + a_prev, b_sum + b_prev
    last = (a_sum[-1], b_sum[-1])
    if transpose_b:
        b_seq, b_sum = b_seq.transpose(-1, -2), b_sum.transpose(-1, -2)
    return a_sum @ b_seq + a_seq @ (b_sum - b_seq), *last


class _StepwiseModule(base.MemoryModule):
    """Single-step logic in ``step``; multi-step mode calls ``sequence`` (default: a loop over the leading axis)."""

    def __init__(self, step_mode: str = "s"):
        super().__init__()
        self.step_mode = step_mode

    def step(self, *xs):
        raise NotImplementedError

    def sequence(self, *xs):
        return torch.stack([self.step(*(x[t] for x in xs)) for t in range(xs[0].shape[0])])

    def forward(self, *xs):
        if self.step_mode == "s":
            return self.step(*xs)
        return self.sequence(*xs)


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

    def _bias_parts(self, x_seq: torch.Tensor) -> Optional[torch.Tensor]:
        """Per-step multiplier ``[T]`` (1 where a bias part is released) for a whole sequence, computed on the device
        without a host read; the two memories become 0-d tensors, which the single-step path accepts as well."""
        T = x_seq.shape[0]
        nz = (x_seq != 0).flatten(1).any(1)
        started = nz.int().cummax(0).values.bool() | torch.as_tensor(self.is_work, device=x_seq.device)
        self.is_work = started[-1]
        if self.spikezip_bias is None:
            return None
        left = torch.as_tensor(self.realize_time, device=x_seq.device)
        release = started & (started.int().cumsum(0) <= left)
        self.realize_time = left - release.sum()
        return release.to(x_seq.dtype).view(T, *([1] * (x_seq.dim() - 1)))


class SpikeZIPLinear(_BiasInParts):
    def __init__(self, linear: nn.Linear, level: int, bias_steps: Optional[int] = None, step_mode: str = "s"):
        super().__init__(linear.bias, level, bias_steps, step_mode)
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.weight = nn.Parameter(linear.weight.detach().clone())

    def step(self, x):
        b = self._bias_part(x)
        return F.linear(x, self.weight, b)

    def sequence(self, x_seq):
        m = self._bias_parts(x_seq)
        y = F.linear(x_seq, self.weight)
        return y if m is None else y + m.view(m.shape[0], *([1] * (y.dim() - 1))) * (self.spikezip_bias / self.bias_steps)


class SpikeZIPConv2d(_BiasInParts):
    def __init__(self, conv: nn.Conv2d, level: int, bias_steps: Optional[int] = None, step_mode: str = "s"):
        super().__init__(conv.bias, level, bias_steps, step_mode)
        self.conv = copy.deepcopy(conv)
        self.conv.bias = None

    def step(self, x):
        b = self._bias_part(x)
        y = self.conv(x)
        return y if b is None else y + b.view(1, -1, 1, 1)

    def sequence(self, x_seq):
        m = self._bias_parts(x_seq)
        T = x_seq.shape[0]
        y = self.conv(x_seq.flatten(0, 1))
        y = y.view(T, -1, *y.shape[1:])
        return y if m is None else y + m.view(T, 1, 1, 1, 1) * (self.spikezip_bias / self.bias_steps).view(1, 1, -1, 1, 1)


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

    def sequence(self, ids_seq):
        y = torch.zeros((*ids_seq.shape, self.embedding.embedding_dim), device=ids_seq.device, dtype=self.embedding.weight.dtype)
        if not self.emitted:
            y[0] = self.embedding(ids_seq[0])
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
        self.is_softmax = bool(getattr(source, "is_softmax", True))      # False: quantised scores divided by the length
        self.attn_if = _neuron(pick("attn_quan"))
        self.after_attn_if = _neuron(pick("after_attn_quan"))
        proj = pick("proj")
        self.proj = SpikeZIPLinear(proj, level) if isinstance(proj, nn.Linear) else None
        self.proj_if = _neuron(pick("proj_quan", "quan_proj")) if self.proj is not None else None
        for name in ("q_sum", "k_sum", "v_sum", "p_sum"):
            self.register_memory(name, None)

    def _heads(self, x):                                  # [..., L, C] -> [..., H, L, D]
        return x.view(*x.shape[:-1], self.num_heads, self.head_dim).transpose(-3, -2)

    def _probabilities(self, scores):
        if self.is_softmax:
            return self.attn_if(self.softmax(scores))
        return self.attn_if(scores) / scores.shape[-1]

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
        p = self._probabilities(scores)
        self.p_sum = self._acc(self.p_sum, p)
        ctx = self.after_attn_if(_matmul_delta(p, v, self.p_sum, self.v_sum))
        out = ctx.transpose(-3, -2).flatten(-2)
        if self.proj is not None:
            out = self.proj_if(self.proj(out))
        return out

    def _children_in(self, mode: str):
        previous = {m: m.step_mode for m in self.modules() if m is not self and hasattr(m, "step_mode")}
        for m in previous:
            m.step_mode = mode
        return previous

    def sequence(self, x_seq):
        """The whole sequence at once: projections with time folded into the batch, the neurons on their sequence
        kernels, and both products as batched increments of the running sums."""
        previous = self._children_in("m")
        try:
            if self.packed:
                q, k, v = self.qkv(x_seq).chunk(3, dim=-1)
            else:
                q, k, v = self.query(x_seq), self.key(x_seq), self.value(x_seq)
            q, k, v = self._heads(self.query_if(q)), self._heads(self.key_if(k)), self._heads(self.value_if(v))
            fresh = not (torch.is_tensor(self.q_sum) and self.q_sum.shape == q.shape[1:])
            scores, self.q_sum, self.k_sum = _matmul_delta_sequence(q, k, None if fresh else self.q_sum, None if fresh else self.k_sum, True)
            p = self._probabilities(scores * self.scale)
            fresh_p = fresh or not (torch.is_tensor(self.p_sum) and self.p_sum.shape == p.shape[1:])
            if fresh_p:
                ctx, self.p_sum, self.v_sum = _matmul_delta_sequence(p, v, None, None)
            else:
                ctx, self.p_sum, self.v_sum = _matmul_delta_sequence(p, v, self.p_sum, self.v_sum)
            out = self.after_attn_if(ctx).transpose(-3, -2).flatten(-2)
            if self.proj is not None:
                out = self.proj_if(self.proj(out))
            return out
        finally:
            for m, mode in previous.items():
                m.step_mode = mode


class SpikeZIPRobertaSelfAttention(SpikeZIPSelfAttention):
    """The attribute-driven wrapper under the reference's name for the RoBERTa layout (``query`` / ``key`` / ``value`` linears,
    ``query_quan`` ... quantisers, ``num_attention_heads``)."""

    def transpose_for_scores(self, x):
        """``[..., L, C] -> [..., H, L, D]`` (the name the RoBERTa attention uses for the head split)."""
        return self._heads(x)


class SpikeZIPViTSelfAttention(SpikeZIPSelfAttention):
    """The same wrapper under the reference's name for the ViT layout (packed ``qkv``, ``quan_q`` ..., ``num_heads``, ``proj``)."""


def _is_qattention(module: nn.Module) -> bool:
    has_proj = getattr(module, "qkv", None) is not None or all(getattr(module, n, None) is not None for n in ("query", "key", "value"))
    has_quan = any(getattr(module, n, None) is not None for n in ("query_quan", "quan_q"))
    has_heads = any(hasattr(module, n) for n in ("num_attention_heads", "num_heads"))
    return has_proj and has_quan and has_heads


class _StepClock(base.MemoryModule):
    """Counts the single steps since the last reset."""

    def __init__(self):
        super().__init__()
        self.register_memory("t", 0)


def _is_vit(model: nn.Module) -> bool:
    return all(hasattr(model, n) for n in ("patch_embed", "cls_token", "pos_embed", "head"))


def _vit_tokens(model: nn.Module, x: torch.Tensor) -> torch.Tensor:
    """Patch tokens ``[..., L, C]`` of images ``[B, C, H, W]`` or ``[T, B, C, H, W]``."""
    embed = model.patch_embed
    proj = getattr(embed, "proj", None)
    y = (proj if proj is not None else embed)(x)
    if y.dim() == x.dim():                                   # still a feature map: [..., C, H', W'] -> [..., L, C]
        y = y.flatten(-2).transpose(-1, -2)
        if proj is not None and hasattr(embed, "norm"):
            y = embed.norm(y)
    return y


def _vit_forward_features(self: nn.Module, x: torch.Tensor) -> torch.Tensor:
    """Class token and position embedding are constants of the ANN: like a bias they enter once, at the first step,
    and later steps carry only what the patch tokens release."""
    if x.dim() not in (4, 5):
        raise ValueError("SpikeZIP ViT forward expects [B, C, H, W] or [T, B, C, H, W].")
    tokens = F.pad(_vit_tokens(self, x), (0, 0, 1, 0))       # a zero token in the class position
    const = self.pos_embed + F.pad(self.cls_token, (0, 0, 0, self.pos_embed.shape[1] - self.cls_token.shape[1]))
    if x.dim() == 5:
        hidden = torch.cat((tokens[:1] + const, tokens[1:]))
    else:
        hidden = tokens + const if self._spikezip_clock.t == 0 else tokens
        self._spikezip_clock.t += 1
    drop = getattr(self, "pos_drop", None)
    if drop is not None:
        hidden = drop(hidden)
    if hasattr(self, "blocks"):
        hidden = self.norm(self.blocks(hidden))
    else:
        hidden = self.norm(hidden + self.attn(self.attn_norm(hidden)))
    return hidden.select(-2, 0)


def _vit_forward(self: nn.Module, x: torch.Tensor) -> torch.Tensor:
    return self.head(self.forward_features(x))


def _install_vit_forward(model: nn.Module) -> None:
    if not hasattr(model, "norm"):
        raise ValueError("SpikeZIP ViT model expects a top-level norm module.")
    if not (hasattr(model, "blocks") or hasattr(model, "attn")):
        raise ValueError("SpikeZIP ViT model expects top-level blocks or attn.")
    if not hasattr(model, "blocks"):
        model.attn_norm = copy.deepcopy(model.norm)          # the single-attention form normalises twice with equal weights
    model._spikezip_clock = _StepClock()
    model.forward_features = types.MethodType(_vit_forward_features, model)
    model.forward = types.MethodType(_vit_forward, model)


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
                cls = SpikeZIPViTSelfAttention if getattr(child, "qkv", None) is not None else SpikeZIPRobertaSelfAttention
                new = cls(child, self._attention_level(child))
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
        if _is_vit(model):
            _install_vit_forward(model)
        model.ann2snn_recipe = "spikezip_tf_qann"
        model.time_steps = self.time_steps
        model.model_family = self.model_family
        return model
