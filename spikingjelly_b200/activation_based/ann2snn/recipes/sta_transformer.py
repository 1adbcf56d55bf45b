"""Training-free conversion of transformers after Spatio-Temporal Approximation (Jiang et al., ICLR 2024).
Parity: ``spikingjelly/activation_based/ann2snn/recipes/sta_transformer.py:1-970``.

Built on the temporal-difference operators of ``ann2snn/operators.py``: the graph rewrite of
:class:`TransformerTDEquivalentRecipe` already makes every Linear / Conv2d / LayerNorm / GELU / attention / matmul node
emit differences of the ANN operator on accumulated inputs.  This recipe adds the two things a transformer graph needs on
top of that:

* **time constants** - floating tensors that the graph reads as attributes and adds to the stream (class token, position
  embedding) must enter the accumulated signal once, so they are emitted at the first step only (:class:`STAConstant`);
  attention masks and weights handed to ``F.linear`` / ``matmul`` are not signals and stay as they are;
* **spike encoders** (``mode="spiking_encoder"``) - after every LayerNorm, GELU and MultiheadAttention output a stateful
  integrate-and-fire encoder with a calibrated per-channel threshold turns the difference signal into integer multiples
  of the threshold (:class:`STASpikeEncoder`).  Thresholds come from forward hooks on the traced ANN during calibration:
  ``max |a| / T`` per channel, or the multiple of it (31 candidates between 1/8 and 2) with the least squared
  quantisation error (``threshold_mode="mse"``).

``mode="equivalent"`` needs no data and reproduces the ANN exactly when the outputs are summed over time.  As in the
reference, ``mode="spiking_affine"`` / ``spike_linear`` / ``spike_conv2d`` are recognised settings that the step-mode
backend rejects.
"""
from __future__ import annotations

import math
import operator
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import fx

from ... import base
from ..operators import TDMultiheadAttention
from .transformer_td_equivalent import TransformerTDEquivalentRecipe

__all__ = ["STATransformerRecipe", "STASpikeEncoder", "STAConstant", "sta_threshold"]

_MODES = ("equivalent", "spiking_encoder", "spiking_affine")
_MASK_KWARGS = frozenset({"attention_mask", "attn_mask", "causal_mask", "decoder_attention_mask", "encoder_attention_mask",
                          "key_padding_mask", "mask", "padding_mask"})
_WEIGHTED_FUNCTIONS = (F.linear, F.conv1d, F.conv2d, F.conv3d)
_MATMULS = (torch.matmul, operator.matmul)
_SEARCH_FACTORS = 31


def sta_threshold(activation: torch.Tensor, time_steps: int, channel_dim: int = -1, mode: str = "mse", eps: float = 1e-6) -> torch.Tensor:
    """Per-channel firing threshold of one calibration batch.  ``"max"``: ``max |a| / T``.  ``"mse"``: among
    ``f * max |a|`` for 31 factors ``f`` in [1/8, 2], the clipping range whose ``T``-level truncating quantiser has the
    least mean squared error on the batch, divided by ``T``."""
    if activation.dim() < 2:
        raise ValueError("STA calibration requires activations with rank >= 2.")
    cd = channel_dim + activation.dim() if channel_dim < 0 else channel_dim
    if not 0 <= cd < activation.dim():
        raise ValueError("channel_dim is out of range.")
    if mode not in ("mse", "max"):
        raise ValueError("STA threshold mode must be 'mse' or 'max'.")
    a = activation.detach().float().movedim(cd, 0).flatten(1)                # [C, n]
    peak = a.abs().amax(dim=1).clamp_min(eps)
    if mode == "max":
        return peak / time_steps
    best = peak.clone()
    best_err = torch.full_like(peak, float("inf"))
    for f in torch.linspace(0.125, 2.0, _SEARCH_FACTORS).tolist():
        rng = (peak * f).clamp_min(eps)
        q = rng[:, None] / time_steps
        err = (a - torch.trunc(a / q) * q).square().mean(dim=1)
        better = err < best_err
        best, best_err = torch.where(better, rng, best), torch.where(better, err, best_err)
    return best / time_steps


class _RunningThreshold:
    """Exponential moving average of :func:`sta_threshold` over the calibration batches (a forward hook)."""

    def __init__(self, time_steps, channel_dim, mode, momentum, eps):
        self.args = (time_steps, channel_dim, mode, eps)
        self.momentum, self.value, self.batches = momentum, None, 0

    def __call__(self, _module, _inputs, output):
        out = output[0] if isinstance(output, (tuple, list)) else output
        if not torch.is_tensor(out):
            raise TypeError("STA observer output must be a tensor.")
        T, cd, mode, eps = self.args
        with torch.no_grad():
            th = sta_threshold(out, T, cd, mode, eps)
            self.value = th if self.value is None else (1 - self.momentum) * self.value.to(th) + self.momentum * th
        self.batches += 1

    def result(self) -> torch.Tensor:
        if self.value is None:
            raise RuntimeError("STA threshold observer did not collect calibration data.")
        if not bool(torch.isfinite(self.value).all()) or bool((self.value <= 0).any()):
            raise ValueError("STA thresholds must be finite positive values.")
        return self.value.detach()


class STASpikeEncoder(base.MemoryModule):
    """Integrate-and-fire re-encoding of a difference signal: the membrane adds the input, emits
    ``trunc(mem / threshold)`` spikes of height ``threshold`` (either sign, several per step) and keeps the rest."""

    def __init__(self, threshold: torch.Tensor, channel_dim: int = -1, step_mode: str = "s") -> None:
        super().__init__()
        self.channel_dim = channel_dim
        self.register_buffer("v_threshold", threshold.detach().clone())
        self.register_memory("mem", None)
        self.step_mode = step_mode

    def _threshold_like(self, x: torch.Tensor) -> torch.Tensor:
        shape = [1] * x.dim()
        shape[self.channel_dim] = self.v_threshold.numel()
        th = self.v_threshold.to(device=x.device, dtype=x.dtype).view(shape)
        return th.clamp_min(torch.finfo(th.dtype).eps)

    def materialize_states(self, inputs, states, step_mode):
        x = inputs[0][0] if step_mode == "m" else inputs[0]
        mem = states[0]
        if not (torch.is_tensor(mem) and mem.shape == x.shape and mem.device == x.device and mem.dtype == x.dtype):
            mem = torch.zeros_like(x)
        return (mem,)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        x = inputs[0]
        th = self._threshold_like(x)
        mem = states[0] + x
        out = torch.trunc(mem / th) * th
        return (out,), (mem - out,)

    def extra_repr(self) -> str:
        return f"channel_dim={self.channel_dim}, step_mode={self.step_mode}"


class STAConstant(base.MemoryModule):
    """A tensor of the graph that belongs to the accumulated signal: the value at the first step after a reset, zeros
    afterwards (a ``[T, ...]`` sequence of that form in multi-step mode)."""

    def __init__(self, value: torch.Tensor, time_steps: int, step_mode: str = "s") -> None:
        super().__init__()
        self.time_steps = time_steps
        if isinstance(value, nn.Parameter):
            self.value = nn.Parameter(value.detach().clone(), requires_grad=value.requires_grad)
        else:
            self.register_buffer("value", value.detach().clone())
        self.register_memory("t", 0)
        self.step_mode = step_mode

    def single_step_forward(self) -> torch.Tensor:
        first = self.t == 0
        self.t = self.t + 1
        return self.value if first else torch.zeros_like(self.value)

    def multi_step_forward(self) -> torch.Tensor:
        seq = torch.zeros_like(self.value).unsqueeze(0).repeat(self.time_steps, *([1] * self.value.dim()))
        if self.t == 0:
            seq[0] = self.value
        self.t = self.t + self.time_steps
        return seq

    def forward(self) -> torch.Tensor:
        return self.multi_step_forward() if self.step_mode == "m" else self.single_step_forward()


# ---------------------------------------------------------------------------------------------------------------------
# settings
# ---------------------------------------------------------------------------------------------------------------------
def _is_number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _is_count(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v > 0


#: (attribute, predicate, message) checked in this order by ``validate``
_SETTING_RULES = (
    ("time_steps", _is_count, "time_steps must be a positive integer."),
    ("mode", lambda v: isinstance(v, str), "mode must be str."),
    ("mode", lambda v: v in _MODES, "mode must be 'equivalent', 'spiking_encoder' or 'spiking_affine'."),
    ("threshold_mode", lambda v: isinstance(v, str), "threshold_mode must be str."),
    ("threshold_mode", lambda v: v in ("mse", "max"), "threshold_mode must be 'mse' or 'max'."),
    ("threshold_scale", _is_number, "threshold_scale must be a positive number."),
    ("threshold_scale", lambda v: v > 0 and math.isfinite(v), "threshold_scale must be positive."),
    ("spike_linear", lambda v: isinstance(v, bool), "spike_linear must be bool."),
    ("spike_conv2d", lambda v: isinstance(v, bool), "spike_conv2d must be bool."),
    ("spike_classifier", lambda v: isinstance(v, bool), "spike_classifier must be bool."),
)
_LATE_RULES = (
    ("momentum", _is_number, "momentum must be a number in [0, 1]."),
    ("momentum", lambda v: 0.0 <= v <= 1.0, "momentum must be in [0, 1]."),
    ("num_calibration_batches", lambda v: v is None or _is_count(v), "num_calibration_batches must be positive or None."),
    ("show_progress", lambda v: isinstance(v, bool), "show_progress must be bool."),
    ("eps", lambda v: _is_number(v) and v > 0 and math.isfinite(v), "eps must be a positive number."),
)


class STATransformerRecipe(TransformerTDEquivalentRecipe):
    """``Converter(recipe=STATransformerRecipe(...))``.  The result is a ``GraphModule`` with ``time_steps`` set; drive it
    with ``functional.set_step_mode`` like any step-mode network (``"s"``: call it once per step; ``"m"``: ``[T, ...]``
    sequences) and sum the outputs over time for the read-out.

    ``dataloader`` yields tensors, ``(input, target)`` pairs, ``((args...), {kwargs})`` pairs or keyword dictionaries; it
    is needed only when something is calibrated (``mode="spiking_encoder"``)."""

    def __init__(self, dataloader: Optional[Iterable] = None, time_steps: int = 32, mode: str = "equivalent", threshold_mode: str = "mse",
                 threshold_scale: float = 1.0, spike_linear: Optional[bool] = None, spike_conv2d: Optional[bool] = None,
                 spike_classifier: bool = False, momentum: float = 0.1, num_calibration_batches: Optional[int] = None,
                 show_progress: bool = False, eps: float = 1e-6) -> None:
        super().__init__(step_mode="m", strict=False)
        self.dataloader, self.time_steps, self.mode = dataloader, time_steps, mode
        self.threshold_mode = threshold_mode.lower() if isinstance(threshold_mode, str) else threshold_mode
        self.threshold_scale = threshold_scale
        self.spike_linear = (mode == "spiking_affine") if spike_linear is None else spike_linear
        self.spike_conv2d = False if spike_conv2d is None else spike_conv2d
        self.spike_classifier, self.momentum = spike_classifier, momentum
        self.num_calibration_batches, self.show_progress, self.eps = num_calibration_batches, show_progress, eps
        self._observers: Dict[str, _RunningThreshold] = {}
        self._hooks: List[Any] = []

    # -- stages -----------------------------------------------------------------------------------------------------
    def validate(self, converter) -> None:
        calibrates = self.mode == "spiking_encoder" or self.spike_linear is True or self.spike_conv2d is True
        if calibrates and self.dataloader is None:
            raise ValueError("STATransformerRecipe requires a dataloader when calibration is enabled. "
                             "Pass dataloader to STATransformerRecipe.")
        for name, ok, message in _SETTING_RULES:
            if not ok(getattr(self, name)):
                raise ValueError(message)
        if self.mode == "spiking_affine" or self.spike_linear or self.spike_conv2d:
            raise ValueError("STATransformerRecipe step-mode backend currently supports only equivalent and spiking_encoder modes "
                             "without spiking affine Linear/Conv2d replacements.")
        for name, ok, message in _LATE_RULES:
            if not ok(getattr(self, name)):
                raise ValueError(message)

    def insert_observers(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        self._drop_hooks()
        self._observers = {}
        if self.mode != "spiking_encoder":
            return fx_model
        modules = dict(fx_model.named_modules())
        for node in fx_model.graph.nodes:
            m = modules.get(node.target) if node.op == "call_module" and isinstance(node.target, str) else None
            if isinstance(m, (nn.LayerNorm, nn.GELU, nn.MultiheadAttention)) and node.target not in self._observers:
                obs = _RunningThreshold(self.time_steps, -1, self.threshold_mode, self.momentum, self.eps)
                self._observers[node.target] = obs
                self._hooks.append(m.register_forward_hook(obs))
        return fx_model

    def calibrate(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        if not self._observers:
            return fx_model
        fx_model.eval()
        batches = self.dataloader
        if self.show_progress:
            from tqdm import tqdm
            batches = tqdm(batches, desc="STA calibration")
        try:
            with torch.no_grad():
                for i, batch in enumerate(batches):
                    if self.num_calibration_batches is not None and i >= self.num_calibration_batches:
                        break
                    args, kwargs = _call_arguments(batch, converter.device)
                    fx_model(*args, **kwargs)
        finally:
            self._drop_hooks()
        return fx_model

    def replace(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        self._drop_hooks()
        modules = dict(fx_model.named_modules())
        encode_after: List[Tuple[fx.Node, torch.Tensor, bool]] = []
        for node in fx_model.graph.nodes:
            m = modules.get(node.target) if node.op == "call_module" and isinstance(node.target, str) else None
            if isinstance(m, nn.MultiheadAttention):
                _check_attention_call(node)
            if node.op == "call_module" and node.target in self._observers:
                encode_after.append((node, self._observers[node.target].result() * self.threshold_scale, isinstance(m, nn.MultiheadAttention)))
        self._wrap_time_constants(fx_model, modules)
        fx_model = super().replace(converter, fx_model)                  # the temporal-difference operators
        for node, threshold, is_attention in encode_after:
            _insert_encoder(fx_model, _attention_output(node) if is_attention else node, threshold)
        fx_model.graph.lint()
        fx_model.recompile()
        return fx_model

    def finalize(self, converter, fx_model: fx.GraphModule) -> nn.Module:
        object.__setattr__(fx_model, "time_steps", self.time_steps)
        return fx_model

    # -- helpers ----------------------------------------------------------------------------------------------------
    def _drop_hooks(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []

    def _wrap_time_constants(self, fx_model: fx.GraphModule, modules: Dict[str, nn.Module]) -> None:
        taken = set(modules)
        n = 0
        for node in list(fx_model.graph.nodes):
            if node.op != "get_attr" or not isinstance(node.target, str):
                continue
            value = fx_model
            for atom in node.target.split("."):
                value = getattr(value, atom)
            if not (torch.is_tensor(value) and value.is_floating_point()) or _is_mask(node, modules) or _is_operator_weight(node):
                continue
            while f"sta_time_constant_{n}" in taken:
                n += 1
            target = f"sta_time_constant_{n}"
            taken.add(target)
            fx_model.add_submodule(target, STAConstant(value, self.time_steps, step_mode="m"))
            with fx_model.graph.inserting_after(node):
                emitted = fx_model.graph.call_module(target, args=())
            node.replace_all_uses_with(emitted)
            fx_model.graph.erase_node(node)


def _to_device(value, device):
    if torch.is_tensor(value):
        return value.to(device)
    if isinstance(value, (tuple, list)):
        return type(value)(_to_device(v, device) for v in value)
    if isinstance(value, dict):
        return {k: _to_device(v, device) for k, v in value.items()}
    return value


def _call_arguments(batch, device) -> Tuple[tuple, dict]:
    """How one calibration batch is passed to the model: ``(args, kwargs)``."""
    if isinstance(batch, dict):
        return (), _to_device(batch, device)
    if isinstance(batch, (tuple, list)):
        if len(batch) == 0:
            raise ValueError("Calibration batch must not be empty.")
        if isinstance(batch[0], (tuple, list)):
            kwargs = _to_device(batch[1], device) if len(batch) > 1 and isinstance(batch[1], dict) else {}
            return tuple(_to_device(v, device) for v in batch[0]), kwargs
        return (_to_device(batch[0], device),), {}
    return (_to_device(batch, device),), {}


def _is_mask(node: fx.Node, modules) -> bool:
    """True when the attribute is used as an attention mask (a static control input, not a signal)."""
    for user in node.users:
        if any(k in _MASK_KWARGS and v is node for k, v in user.kwargs.items()):
            return True
        args = tuple(user.args)
        if user.op == "call_module" and isinstance(modules.get(user.target), (nn.MultiheadAttention, TDMultiheadAttention)):
            if (len(args) > 3 and args[3] is node) or (len(args) > 5 and args[5] is node):
                return True
        if user.op == "call_function" and user.target is F.scaled_dot_product_attention and len(args) > 3 and args[3] is node:
            return True
    return False


def _is_operator_weight(node: fx.Node) -> bool:
    """True when the attribute is the weight of a functional linear / convolution or an operand of a matmul."""
    for user in node.users:
        if user.op != "call_function":
            continue
        if user.target in _WEIGHTED_FUNCTIONS and ((len(user.args) > 1 and user.args[1] is node) or user.kwargs.get("weight") is node):
            return True
        if user.target in _MATMULS and (node in tuple(user.args) or user.kwargs.get("input") is node or user.kwargs.get("other") is node):
            return True
    return False


def _check_attention_call(node: fx.Node) -> None:
    need = node.kwargs["need_weights"] if "need_weights" in node.kwargs else (node.args[4] if len(node.args) > 4 else None)
    if need is True:
        raise ValueError("STATransformerRecipe step-mode backend requires MultiheadAttention calls with need_weights=False. "
                         "Use a custom online wrapper when attention weights are required.")
    if need not in (None, False):
        raise ValueError("STATransformerRecipe step-mode backend only supports literal need_weights=False for MultiheadAttention.")
    if need is None:
        for user in node.users:
            if user.op == "call_function" and user.target is operator.getitem and len(user.args) >= 2 and user.args[1] == 1 and user.users:
                raise ValueError("STATransformerRecipe step-mode backend does not support using MultiheadAttention attention "
                                 "weights. Pass need_weights=False.")


def _attention_output(node: fx.Node) -> fx.Node:
    for user in node.users:
        if user.op == "call_function" and user.target is operator.getitem and len(user.args) >= 2 and user.args[1] == 0:
            return user
    raise ValueError("STATransformerRecipe step-mode backend with spiking_encoder requires MultiheadAttention output to be "
                     "unpacked before use.")


def _insert_encoder(fx_model: fx.GraphModule, node: fx.Node, threshold: torch.Tensor) -> str:
    existing = dict(fx_model.named_modules())
    stem = (node.target if isinstance(node.target, str) else node.name).replace(".", "_") + "_sta_encoder"
    target, k = stem, 0
    while target in existing:
        k += 1
        target = f"{stem}_{k}"
    fx_model.add_submodule(target, STASpikeEncoder(threshold, channel_dim=-1, step_mode="m"))
    with fx_model.graph.inserting_after(node):
        enc = fx_model.graph.call_module(target, args=(node,))
    for user in list(node.users):
        if user is not enc:
            user.replace_input_with(node, enc)
    return target
