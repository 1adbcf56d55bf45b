"""Post-training conversion of a Hugging Face Qwen2 causal language model into an offline multi-step TD / SNN hybrid
(parity: ``spikingjelly/activation_based/ann2snn/recipes/qwen2.py:39-1360``).

The converted model keeps an explicit time axis ``[T, B, S, H]`` through every decoder layer.  Linear maps, RMSNorm, SiLU,
the gate * up product and attention are temporal-difference operators (``ann2snn/operators.py``); at five places per
layer - the embedding output, rotated queries, rotated keys, values and the MLP intermediate - the accumulated signal is
re-encoded by a :class:`~..qcfs.SignedQCFSSequenceEncoder` whose per-channel step was calibrated on data:

* ``encoding_mode="signed_if"`` (default): positive / negative integrate-and-fire populations emit the ``T``-step spike
  sequence;
* ``"qcfs_sg"``: the quantised value is reconstructed in one step with a surrogate gradient (for post-training);
* ``"exact_td"``: no quantisation, to check that the temporal-difference graph reproduces the source model.

Calibration (:func:`calibrate_qwen2_snn`) hooks the source model, never keeps whole activations, and reduces each
observed tensor to a per-channel bound: the running maximum (``quantile == 1``) or a quantile over a fixed-size reservoir
of token rows drawn by priority sampling.  ``scale = bound / calibration_levels``.

Decoding is greedy with a KV cache of accumulated keys / values; neuron state is reset before every chunk.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, fields
from types import SimpleNamespace
from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..operators import SNNElementWiseProduct, TDRMSNorm, TDScaledDotProductAttention, TDSiLU, _td_module_from_ann
from ..qcfs import SignedQCFSSequenceEncoder
from .base import ModuleConversionRecipe

__all__ = ["Qwen2SNNConfig", "Qwen2SNNCalibration", "Qwen2SNNModel", "Qwen2SNNRecipe", "calibrate_qwen2_snn"]

#: the four re-encoding points of a decoder layer
SCALE_NAMES = ("query", "key", "value", "mlp")
ENCODING_MODES = ("signed_if", "qcfs_sg", "exact_td")


def _plain_int(value, name: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool):
        raise TypeError(f"{name} must be an integer.")
    return value


@dataclass
class Qwen2SNNConfig:
    """``time_steps``: length of the time axis and range of representable spike counts; ``calibration_levels`` (at most
    ``time_steps``): the per-channel quantisation step is ``bound / calibration_levels``; ``calibration_quantile`` in
    (0, 1]: which quantile of ``|activation|`` is the bound; reservoir size and seed: the priority sample the quantile is
    taken over; ``neuron_backend``: backend of the encoder neurons (``"torch"``, ``"triton"`` as an alias kept for
    configurations written for the reference, or ``"cuda"``)."""
    time_steps: int = 32
    calibration_levels: int = 16
    calibration_quantile: float = 1.0
    calibration_reservoir_size: int = 4096
    calibration_seed: int = 20260719
    neuron_backend: str = "torch"

    def __post_init__(self) -> None:
        if _plain_int(self.time_steps, "time_steps") <= 0:
            raise ValueError("time_steps must be positive.")
        if not 0 < _plain_int(self.calibration_levels, "calibration_levels") <= self.time_steps:
            raise ValueError("calibration_levels must lie in [1, time_steps].")
        if not 0.0 < float(self.calibration_quantile) <= 1.0:
            raise ValueError("calibration_quantile must lie in (0, 1].")
        if _plain_int(self.calibration_reservoir_size, "calibration_reservoir_size") <= 0:
            raise ValueError("calibration_reservoir_size must be positive.")
        _plain_int(self.calibration_seed, "calibration_seed")
        if self.neuron_backend not in ("torch", "triton", "cuda"):
            raise ValueError("neuron_backend must be 'torch' or 'triton'.")


_SHARED_FIELDS = ("time_steps", "calibration_levels", "calibration_quantile", "calibration_reservoir_size", "calibration_seed")


@dataclass(frozen=True)
class Qwen2SNNCalibration:
    """Per-channel encoder steps: one vector for the embedding output and four per decoder layer, with the settings they
    were computed under.  :meth:`state_dict` holds tensors and plain Python values only (``torch.load(...,
    weights_only=True)`` reads it back)."""
    input_scale: torch.Tensor
    layer_scales: Tuple[Mapping[str, torch.Tensor], ...]
    time_steps: int
    calibration_levels: int
    calibration_quantile: float
    calibration_reservoir_size: int
    calibration_seed: int
    valid_token_count: int

    def state_dict(self) -> Dict[str, object]:
        tensors = {"input": self.input_scale.detach().cpu()}
        for i, group in enumerate(self.layer_scales):
            tensors.update({f"layer.{i}.{name}": value.detach().cpu() for name, value in group.items()})
        state: Dict[str, object] = {name: getattr(self, name) for name in _SHARED_FIELDS}
        state["valid_token_count"] = self.valid_token_count
        state["tensors"] = tensors
        return state

    @classmethod
    def from_state_dict(cls, state: Mapping[str, object]) -> "Qwen2SNNCalibration":
        tensors = state.get("tensors")
        if not isinstance(tensors, Mapping) or not isinstance(tensors.get("input"), torch.Tensor):
            raise ValueError("Calibration state requires a tensors mapping with an 'input' entry.")
        groups: Dict[int, Dict[str, torch.Tensor]] = {}
        for key, value in tensors.items():
            if key == "input":
                continue
            parts = str(key).split(".")
            if len(parts) != 3 or parts[0] != "layer" or not parts[1].isdigit() or parts[2] not in SCALE_NAMES:
                raise ValueError(f"Unexpected calibration tensor key {key!r}.")
            if not isinstance(value, torch.Tensor):
                raise ValueError(f"Calibration entry {key!r} is not a tensor.")
            groups.setdefault(int(parts[1]), {})[parts[2]] = value
        if sorted(groups) != list(range(len(groups))):
            raise ValueError("Calibration layer indices must be contiguous from zero.")
        for i, group in groups.items():
            if set(group) != set(SCALE_NAMES):
                raise ValueError(f"Calibration layer {i} must hold exactly the scales {SCALE_NAMES}.")
        meta = {}
        for f in fields(cls):
            if f.name in ("input_scale", "layer_scales"):
                continue
            if f.name not in state:
                raise ValueError(f"Calibration state lacks {f.name!r}.")
            meta[f.name] = state[f.name]
        return cls(input_scale=tensors["input"], layer_scales=tuple(groups[i] for i in range(len(groups))), **meta)


class _ChannelBound:
    """Running per-channel bound of ``|activation|`` over the valid tokens of the calibration set."""

    def __init__(self, quantile: float, reservoir: int, seed: int) -> None:
        self.quantile, self.reservoir = quantile, reservoir
        self.rows: Optional[torch.Tensor] = None            # [1, C] running maximum, or [n <= reservoir, C] sampled rows
        self.priority: Optional[torch.Tensor] = None
        self.rng = torch.Generator(device="cpu").manual_seed(seed)
        self.valid_token_count = 0

    def update(self, activation: torch.Tensor, mask: torch.Tensor) -> None:
        rows = activation.detach()[mask.to(torch.bool)]
        if rows.numel() == 0:
            raise ValueError("Qwen2 calibration requires at least one valid token.")
        self.valid_token_count += int(rows.shape[0])
        if self.quantile == 1.0:
            top = rows.abs().amax(0, keepdim=True)
            self.rows = top if self.rows is None else torch.maximum(self.rows, top)
            return
        # priority sampling: every row draws a uniform key, the `reservoir` largest keys seen so far stay
        keys = torch.rand(rows.shape[0], generator=self.rng)
        keys, pick = keys.topk(min(self.reservoir, rows.shape[0]))
        kept = rows.index_select(0, pick.to(rows.device)).abs().to("cpu", torch.float32)
        if self.rows is not None:
            kept, keys = torch.cat((self.rows, kept)), torch.cat((self.priority, keys))
        self.priority, order = keys.topk(min(self.reservoir, kept.shape[0]))
        self.rows = kept.index_select(0, order)

    def scale(self, levels: int) -> torch.Tensor:
        if self.rows is None:
            raise RuntimeError("Qwen2 calibration observer received no values.")
        bound = self.rows.squeeze(0) if self.quantile == 1.0 else torch.quantile(self.rows, self.quantile, dim=0)
        return bound.clamp_min(1e-6) / levels


# ---------------------------------------------------------------------------------------------------------------------
# tensor helpers ([..., S, H] <-> [..., heads, S, D])
# ---------------------------------------------------------------------------------------------------------------------
def _to_heads(x: torch.Tensor, heads: int, width: int) -> torch.Tensor:
    return x.view(*x.shape[:-1], heads, width).transpose(-3, -2)


def _from_heads(x: torch.Tensor) -> torch.Tensor:
    return x.transpose(-3, -2).flatten(-2)


def _rotate(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    def half_turn(v):
        h = v.shape[-1] // 2
        return torch.cat((-v[..., h:], v[..., :h]), dim=-1)
    cos, sin = cos.unsqueeze(-3), sin.unsqueeze(-3)
    while cos.dim() < q.dim():
        cos, sin = cos.unsqueeze(0), sin.unsqueeze(0)
    return q * cos + half_turn(q) * sin, k * cos + half_turn(k) * sin


def _share_kv(x: torch.Tensor, groups: int) -> torch.Tensor:
    """``[T, B, kv_heads, S, D]`` -> ``[T, B, kv_heads * groups, S, D]`` (grouped-query attention)."""
    if groups == 1:
        return x
    T, B, H, S, D = x.shape
    return x[:, :, :, None].expand(T, B, H, groups, S, D).reshape(T, B, H * groups, S, D)


def _first_step_sequence(value: torch.Tensor, T: int) -> torch.Tensor:
    seq = value.new_zeros((T, *value.shape))
    seq[0] = value
    return seq


def _attention_mask(mask: torch.Tensor, q_len: int, past: int) -> torch.Tensor:
    total = past + q_len
    if mask.dim() != 2 or mask.shape[1] != total:
        raise ValueError("attention_mask length must equal past_length + query_length.")
    q_pos = torch.arange(past, total, device=mask.device).unsqueeze(1)
    k_pos = torch.arange(total, device=mask.device).unsqueeze(0)
    return (k_pos <= q_pos)[None, None] & mask[:, None, None, :].to(torch.bool)


def _td_norm(source: nn.Module) -> TDRMSNorm:
    weight = getattr(source, "weight", None)
    if not isinstance(weight, torch.Tensor):
        raise TypeError("Qwen2 RMSNorm must expose tensor weight.")
    eps = getattr(source, "variance_epsilon", getattr(source, "eps", None))
    norm = TDRMSNorm(weight.shape, eps=eps, device=weight.device, dtype=weight.dtype)
    with torch.no_grad():
        norm.weight.copy_(weight)
    norm.weight.requires_grad = weight.requires_grad
    return norm.train(source.training)


def _decoder_layers(model: nn.Module) -> Sequence[nn.Module]:
    layers = getattr(getattr(model, "model", None), "layers", None)
    if not isinstance(layers, (nn.ModuleList, list, tuple)):
        raise TypeError("Qwen2 model must expose model.layers.")
    return layers


def _check_source(model: nn.Module) -> Sequence[nn.Module]:
    cfg = getattr(model, "config", None)
    if cfg is None or getattr(cfg, "model_type", None) != "qwen2":
        raise TypeError("Qwen2SNNRecipe requires a Hugging Face Qwen2 causal LM.")
    if bool(getattr(cfg, "use_sliding_window", False)):
        raise ValueError("Qwen2 sliding-window attention is not supported.")
    if bool(getattr(cfg, "use_mrope", False)):
        raise ValueError("Qwen2 MRoPE is not supported.")
    if getattr(cfg, "hidden_act", "silu") != "silu":
        raise ValueError("Qwen2SNNRecipe requires hidden_act='silu'.")
    if model.training:
        raise ValueError("Qwen2SNNRecipe requires evaluation-mode source; call eval().")
    layers = _decoder_layers(model)
    if len(layers) != int(cfg.num_hidden_layers):
        raise ValueError("Qwen2 config and concrete decoder layer count disagree.")
    return layers


class _KVCache:
    """Accumulated (time-summed) keys and values of every layer, ``[B, kv_heads, S, D]`` each."""

    def __init__(self, n_layers: int) -> None:
        self.entries: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = [None] * n_layers

    def append(self, i: int, key: torch.Tensor, value: torch.Tensor) -> None:
        old = self.entries[i]
        if old is not None:
            key, value = torch.cat((old[0], key), dim=2), torch.cat((old[1], value), dim=2)
        self.entries[i] = (key.detach(), value.detach())

    def get_seq_length(self) -> int:
        first = self.entries[0] if self.entries else None
        return 0 if first is None else int(first[0].shape[2])

    def reorder_cache(self, indices: torch.Tensor) -> None:
        self.entries = [None if e is None else (e[0].index_select(0, indices), e[1].index_select(0, indices)) for e in self.entries]

    def storage_summary(self) -> Dict[str, object]:
        logical, storages, shapes = 0, {}, []
        for e in self.entries:
            if e is None:
                shapes.append(None)
                continue
            shapes.append({"key": list(e[0].shape), "value": list(e[1].shape)})
            for t in e:
                logical += t.numel() * t.element_size()
                st = t.untyped_storage()
                storages[st.data_ptr()] = st.nbytes()
        return {"representation": "accumulated_kv", "layers": shapes, "stored_cache_logical_bytes": logical,
                "stored_cache_unique_storage_bytes": sum(storages.values()), "theoretical_cache_bytes": logical,
                "temporal_prefix_materialization_bytes": 0}


class _DecoderLayer(nn.Module):
    def __init__(self, source: nn.Module, scales: Mapping[str, torch.Tensor], T: int, backend: str, index: int) -> None:
        super().__init__()
        attn, mlp = source.self_attn, source.mlp
        self.index, self.time_steps = index, T
        self.heads, self.kv_heads = int(attn.config.num_attention_heads), int(attn.config.num_key_value_heads)
        self.head_dim, self.kv_groups = int(attn.head_dim), int(attn.num_key_value_groups)
        self.input_layernorm, self.post_attention_layernorm = _td_norm(source.input_layernorm), _td_norm(source.post_attention_layernorm)
        for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
            setattr(self, name, _td_module_from_ann(getattr(attn, name)))
        for name in ("gate_proj", "up_proj", "down_proj"):
            setattr(self, name, _td_module_from_ann(getattr(mlp, name)))
        self.sdpa = TDScaledDotProductAttention(scale=float(attn.scaling))
        self.act, self.product = TDSiLU(), SNNElementWiseProduct()
        self.encoders = nn.ModuleDict({name: SignedQCFSSequenceEncoder(scales[name], T, neuron_backend=backend, name=f"layer.{index}.{name}")
                                       for name in SCALE_NAMES})

    def _recode(self, name: str, seq: torch.Tensor, mode: str, mask: torch.Tensor) -> torch.Tensor:
        total = seq.sum(0)
        if mode == "exact_td":
            return _first_step_sequence(total, self.time_steps)
        if mode == "qcfs_sg":
            return _first_step_sequence(self.encoders[name].reconstruct(total), self.time_steps)
        return self.encoders[name].encode(total, mask)

    def _attend(self, q, k, v, attn_mask, cache: Optional[_KVCache]):
        past = None
        if cache is not None:
            past = cache.entries[self.index]
            cache.append(self.index, k.sum(0), v.sum(0))
        dtype = q.dtype
        with torch.amp.autocast(q.device.type, enabled=False):
            q, k, v = q.float(), _share_kv(k.float(), self.kv_groups), _share_kv(v.float(), self.kv_groups)
            if past is None:
                out = self.sdpa(q, k, v, attn_mask)
            else:
                # the cached prefix belongs to the accumulated signal: it enters at the first step only
                pk = past[0].float().repeat_interleave(self.kv_groups, dim=1)
                pv = past[1].float().repeat_interleave(self.kv_groups, dim=1)
                zk, zv = torch.zeros_like(pk), torch.zeros_like(pv)
                out = torch.stack([self.sdpa.single_step_forward(q[t], torch.cat((pk if t == 0 else zk, k[t]), dim=2),
                                                                 torch.cat((pv if t == 0 else zv, v[t]), dim=2), attn_mask)
                                   for t in range(q.shape[0])])
        return _from_heads(out.to(dtype))

    def forward(self, hidden, *, cos, sin, attention_mask, value_mask, encoding_mode, cache):
        h = self.input_layernorm(hidden)
        q = _to_heads(self.q_proj(h), self.heads, self.head_dim)
        k = _to_heads(self.k_proj(h), self.kv_heads, self.head_dim)
        v = _to_heads(self.v_proj(h), self.kv_heads, self.head_dim)
        q, k = _rotate(q, k, cos, sin)
        q = _to_heads(self._recode("query", _from_heads(q), encoding_mode, value_mask), self.heads, self.head_dim)
        k = _to_heads(self._recode("key", _from_heads(k), encoding_mode, value_mask), self.kv_heads, self.head_dim)
        v = _to_heads(self._recode("value", _from_heads(v), encoding_mode, value_mask), self.kv_heads, self.head_dim)
        hidden = hidden + self.o_proj(self._attend(q, k, v, attention_mask, cache))
        h = self.post_attention_layernorm(hidden)
        mid = self.product(self.act(self.gate_proj(h)), self.up_proj(h))
        return hidden + self.down_proj(self._recode("mlp", mid, encoding_mode, value_mask))


# TDScaledDotProductAttention.single_step_forward takes (q, k, v); the mask travels as an attribute
def _sdpa_single_step(self, q, k, v, attn_mask=None):
    self.attn_mask = attn_mask
    try:
        return super(TDScaledDotProductAttention, self).single_step_forward(q, k, v)
    finally:
        self.attn_mask = None


class _MaskedStepSDPA(TDScaledDotProductAttention):
    single_step_forward = _sdpa_single_step


class Qwen2SNNModel(nn.Module):
    """The converted model.  ``forward(input_ids, attention_mask=None, *, position_ids=None, encoding_mode=None,
    past_key_values=None, use_cache=False)`` returns a namespace with ``logits`` ``[B, S, vocab]`` (read out from the
    time-summed last hidden state in fp32) and ``past_key_values``."""
    temporal_layout = "[T,B,S,H]"
    execution_schedule = "layerwise_offline_multistep"
    online_inference = False

    def __init__(self, source: nn.Module, calibration: Qwen2SNNCalibration, conversion: Qwen2SNNConfig) -> None:
        super().__init__()
        inner = source.model
        self.config, self.time_steps = source.config, conversion.time_steps
        self.embed_tokens = copy.deepcopy(inner.embed_tokens)
        self.rotary_emb = inner.rotary_emb
        self.layers = nn.ModuleList(_DecoderLayer(layer, calibration.layer_scales[i], conversion.time_steps, conversion.neuron_backend, i)
                                    for i, layer in enumerate(inner.layers))
        for layer in self.layers:
            layer.sdpa.__class__ = _MaskedStepSDPA
        self.norm = _td_norm(inner.norm)
        self.lm_head = _td_module_from_ann(source.lm_head)
        if bool(getattr(self.config, "tie_word_embeddings", False)):
            self.lm_head.weight = self.embed_tokens.weight
        self.input_encoder = SignedQCFSSequenceEncoder(calibration.input_scale, conversion.time_steps,
                                                       neuron_backend=conversion.neuron_backend, name="model.input")

    # -- introspection ------------------------------------------------------------------------------------------------
    def signed_encoders(self) -> Tuple[SignedQCFSSequenceEncoder, ...]:
        return (self.input_encoder, *(layer.encoders[name] for layer in self.layers for name in SCALE_NAMES))

    def set_collect_statistics(self, enabled: bool) -> None:
        for enc in self.signed_encoders():
            enc.collect_statistics = bool(enabled)

    def encoder_statistics(self) -> Tuple[Dict[str, object], ...]:
        return tuple(enc.statistics() for enc in self.signed_encoders())

    def structure_summary(self) -> Dict[str, object]:
        kinds: Dict[str, int] = {}
        for m in self.modules():
            kinds[type(m).__name__] = kinds.get(type(m).__name__, 0) + 1
        return {"temporal_layout": self.temporal_layout, "execution_schedule": self.execution_schedule,
                "online_inference": self.online_inference, "time_steps": self.time_steps, "decoder_layers": len(self.layers),
                "signed_encoders": len(self.signed_encoders()), "module_types": dict(sorted(kinds.items()))}

    @property
    def device(self) -> torch.device:
        return self.embed_tokens.weight.device

    def get_input_embeddings(self) -> nn.Embedding:
        return self.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def tie_weights(self) -> None:
        if bool(getattr(self.config, "tie_word_embeddings", False)):
            self.lm_head.weight = self.embed_tokens.weight

    # -- inference ----------------------------------------------------------------------------------------------------
    def _reset_state(self) -> None:
        for m in self.modules():
            reset = getattr(m, "reset", None)
            if callable(reset):
                reset()

    def generate(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None, *, max_new_tokens: int,
                 do_sample: bool = False, num_beams: int = 1, **_: object) -> torch.Tensor:
        """Greedy decoding with the KV cache: ``[B, S]`` -> ``[B, S + max_new_tokens]``."""
        if do_sample or num_beams != 1:
            raise ValueError("Converted Qwen2 supports deterministic greedy generation only.")
        if max_new_tokens < 0:
            raise ValueError("max_new_tokens must be non-negative.")
        with torch.inference_mode():
            tokens = input_ids
            mask = torch.ones_like(input_ids) if attention_mask is None else attention_mask
            cache = None
            for i in range(max_new_tokens):
                self._reset_state()
                out = self(input_ids=tokens if i == 0 else tokens[:, -1:], attention_mask=mask, past_key_values=cache, use_cache=True)
                cache = out.past_key_values
                nxt = out.logits[:, -1].argmax(-1, keepdim=True)
                tokens, mask = torch.cat((tokens, nxt), dim=1), torch.cat((mask, torch.ones_like(nxt)), dim=1)
            return tokens

    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None, *, position_ids: Optional[torch.Tensor] = None,
                encoding_mode: Optional[str] = None, past_key_values: Optional[_KVCache] = None, use_cache: bool = False,
                **_: object) -> SimpleNamespace:
        mode = encoding_mode or "signed_if"
        if mode not in ENCODING_MODES:
            raise ValueError(f"Unsupported encoding_mode={mode!r}.")
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        if past_key_values is not None and not use_cache:
            raise ValueError("past_key_values requires use_cache=True.")
        past = 0 if past_key_values is None else past_key_values.get_seq_length()
        if use_cache and past_key_values is None:
            past_key_values = _KVCache(len(self.layers))
        S = input_ids.shape[1]
        emb = self.embed_tokens(input_ids)
        if position_ids is None:
            # positions count valid tokens, so left padding and cache continuation both come out right
            position_ids = attention_mask.to(torch.long).cumsum(-1) - 1
            position_ids.masked_fill_(~attention_mask.to(torch.bool), 0)
            position_ids = position_ids[:, -S:]
        elif tuple(position_ids.shape) != tuple(input_ids.shape):
            raise ValueError("position_ids shape must match input_ids shape.")
        position_ids = position_ids.to(device=input_ids.device, dtype=torch.long)
        cos, sin = self.rotary_emb(emb, position_ids)
        allowed = _attention_mask(attention_mask, S, past)
        value_mask = attention_mask[:, -S:]
        if mode == "exact_td":
            hidden = _first_step_sequence(emb, self.time_steps)
        elif mode == "qcfs_sg":
            hidden = _first_step_sequence(self.input_encoder.reconstruct(emb), self.time_steps)
        else:
            hidden = self.input_encoder.encode(emb, value_mask)
        for layer in self.layers:
            hidden = layer(hidden, cos=cos, sin=sin, attention_mask=allowed, value_mask=value_mask, encoding_mode=mode, cache=past_key_values)
        hidden = self.norm(hidden)
        with torch.amp.autocast(hidden.device.type, enabled=False):
            bias = self.lm_head.bias
            logits = F.linear(hidden.sum(0).float(), self.lm_head.weight.float(), None if bias is None else bias.float())
        return SimpleNamespace(logits=logits, past_key_values=past_key_values)


def calibrate_qwen2_snn(model: nn.Module, calibration_batches: Iterable[Mapping[str, torch.Tensor]], config: Qwen2SNNConfig) -> Qwen2SNNCalibration:
    """Run ``calibration_batches`` (mappings with ``input_ids`` and ``attention_mask``, already on the model's device)
    through the evaluation-mode source model and return the per-channel encoder steps.  Hooks recompute the rotated
    queries / keys, the values and the MLP intermediate from each module's input, so no full activation is stored."""
    layers = list(_check_source(model))
    make = lambda: _ChannelBound(config.calibration_quantile, config.calibration_reservoir_size, config.calibration_seed)
    at_input, per_layer = make(), [{name: make() for name in SCALE_NAMES} for _ in layers]
    current = {}

    def on_embedding(_m, _inputs, output):
        at_input.update(output, current["mask"])

    def on_attention(i):
        def hook(module, _args, kwargs):
            h = kwargs["hidden_states"]
            d, nh, nkv = int(module.head_dim), int(module.config.num_attention_heads), int(module.config.num_key_value_heads)
            q, k, v = _to_heads(module.q_proj(h), nh, d), _to_heads(module.k_proj(h), nkv, d), _to_heads(module.v_proj(h), nkv, d)
            q, k = _rotate(q, k, *kwargs["position_embeddings"])
            for name, t in (("query", q), ("key", k), ("value", v)):
                per_layer[i][name].update(_from_heads(t), current["mask"])
        return hook

    def on_mlp(i):
        def hook(module, inputs):
            h = inputs[0]
            per_layer[i]["mlp"].update(module.act_fn(module.gate_proj(h)) * module.up_proj(h), current["mask"])
        return hook

    handles = [model.model.embed_tokens.register_forward_hook(on_embedding)]
    for i, layer in enumerate(layers):
        handles.append(layer.self_attn.register_forward_pre_hook(on_attention(i), with_kwargs=True))
        handles.append(layer.mlp.register_forward_pre_hook(on_mlp(i)))
    try:
        with torch.no_grad():
            for batch in calibration_batches:
                ids, mask = batch.get("input_ids"), batch.get("attention_mask")
                if not isinstance(ids, torch.Tensor) or not isinstance(mask, torch.Tensor):
                    raise TypeError("Calibration batches require tensor input_ids and attention_mask.")
                current["mask"] = mask
                model(input_ids=ids, attention_mask=mask, use_cache=False, return_dict=True)
    finally:
        for h in handles:
            h.remove()
    L = config.calibration_levels
    return Qwen2SNNCalibration(input_scale=at_input.scale(L), layer_scales=tuple({n: o.scale(L) for n, o in g.items()} for g in per_layer),
                               valid_token_count=at_input.valid_token_count, **{name: getattr(config, name) for name in _SHARED_FIELDS})


class Qwen2SNNRecipe(ModuleConversionRecipe):
    """``ModuleConverter(Qwen2SNNRecipe(calibration, config)).convert(qwen2_causal_lm.eval())`` -> :class:`Qwen2SNNModel`."""

    def __init__(self, calibration: Qwen2SNNCalibration, config: Qwen2SNNConfig) -> None:
        self.calibration, self.config = calibration, config

    def validate(self, converter) -> None:
        for name in _SHARED_FIELDS:
            if getattr(self.calibration, name) != getattr(self.config, name):
                raise ValueError(f"Calibration {name} does not match config.")

    def convert_module(self, converter, ann: nn.Module) -> Qwen2SNNModel:
        if len(_check_source(ann)) != len(self.calibration.layer_scales):
            raise ValueError("Calibration layer count does not match Qwen2 model.")
        return Qwen2SNNModel(ann, self.calibration, self.config).eval()
