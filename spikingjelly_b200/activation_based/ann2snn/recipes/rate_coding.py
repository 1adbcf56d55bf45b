"""Rate-coding conversion (Rueckauer et al. 2017): fold BatchNorm into convolutions, observe the scale
of every ReLU output on calibration data, and replace each ReLU by ``scale down -> IF neuron -> scale up``.
Layer-wise (one scalar per ReLU) or channel-wise thresholds; max / percentile / fraction-of-max norms.
Parity: ``spikingjelly/activation_based/ann2snn/recipes/rate_coding.py:41-687``."""
from __future__ import annotations

import math
from typing import Dict, Iterable, Optional, Union

import torch
import torch.nn as nn
from torch import fx
from torch.nn.utils.fusion import fuse_conv_bn_eval

from ... import neuron
from ..factories import NeuronFactory
from ..modules import ChannelVoltageScaler, VoltageHook, VoltageScaler, _scale_statistic
from .base import ConversionRecipe
from .step_mode_adapters import adapt_step_mode_graph

__all__ = ["RateCodingRecipe", "ChannelVoltageHook", "validate_rate_coding_mode"]

_BAD_MODE = "You have used a non-defined VoltageScale Method."
_INPUT_KEYS = ("input", "image", "images", "img", "x", "data", "pixel_values")


def validate_rate_coding_mode(mode) -> None:
    if isinstance(mode, str):
        if mode and mode[-1] == "%":
            try:
                ok = 0.0 <= float(mode[:-1]) <= 100.0
            except ValueError as exc:
                raise NotImplementedError(_BAD_MODE) from exc
            if not ok:
                raise NotImplementedError(_BAD_MODE)
        elif mode.lower() != "max":
            raise NotImplementedError(_BAD_MODE)
    elif isinstance(mode, (int, float)) and not isinstance(mode, bool):
        if not 0 < mode <= 1:
            raise NotImplementedError(_BAD_MODE)
    else:
        raise NotImplementedError(_BAD_MODE)


def _extract_batch_input(data, _inside=False):
    """The model input of a dataloader item: a tensor, the first element of ``(x, y)``, or a known key of a dict."""
    if isinstance(data, torch.Tensor):
        return data
    if isinstance(data, (list, tuple)):
        if not data:
            raise ValueError("Batch data is an empty list or tuple.")
        if len(data) == 1:
            return _extract_batch_input(data[0], _inside)
        return data if _inside else _extract_batch_input(data[0], not isinstance(data[0], dict))
    if isinstance(data, dict):
        if not data:
            raise ValueError("Batch data is an empty dictionary.")
        if _inside:
            return data
        for k in _INPUT_KEYS:
            if k in data:
                return _extract_batch_input(data[k], True)
        if len(data) != 1:
            raise ValueError("Batch dictionaries with multiple fields must contain one of 'input', 'image', 'images', 'img', 'x', "
                             "'data', or 'pixel_values'.")
        return _extract_batch_input(next(iter(data.values())), True)
    return data


def _is_relu(node: fx.Node, modules) -> bool:
    return node.op == "call_module" and isinstance(node.target, str) and type(modules.get(node.target)) is nn.ReLU


def _insert(fx_model, target, after, module, args):
    fx_model.add_submodule(target, module)
    with fx_model.graph.inserting_after(after):
        return fx_model.graph.call_module(target, args=args)


def _fuse_conv_bn(fx_model: fx.GraphModule, fuse_flag: bool = True) -> fx.GraphModule:
    if not fuse_flag:
        return fx_model
    modules = dict(fx_model.named_modules())
    pairs = ((nn.Conv1d, nn.BatchNorm1d), (nn.Conv2d, nn.BatchNorm2d), (nn.Conv3d, nn.BatchNorm3d))
    for node in list(fx_model.graph.nodes):
        if node.op != "call_module" or not node.args or not isinstance(node.args[0], fx.Node):
            continue
        src = node.args[0]
        if src.op != "call_module" or len(src.users) > 1:
            continue
        conv, bn = modules.get(src.target), modules.get(node.target)
        if any(isinstance(conv, c) and isinstance(bn, b) for c, b in pairs):
            fused = fuse_conv_bn_eval(conv, bn)
            parent, _, child = src.target.rpartition(".")
            setattr(fx_model.get_submodule(parent) if parent else fx_model, child, fused)
            modules[src.target] = fused
            node.replace_all_uses_with(src)
            fx_model.graph.erase_node(node)
    fx_model.graph.lint()
    fx_model.delete_all_unused_submodules()
    fx_model.recompile()
    return fx_model


class ChannelVoltageHook(nn.Module):
    """Per-channel version of ``VoltageHook`` (statistic of the non-negative part, floored at ``eps``)."""

    def __init__(self, mode="Max", momentum: float = 0.1, channel_dim: int = 1, eps: float = 1e-6) -> None:
        super().__init__()
        self.mode, self.momentum, self.channel_dim, self.eps = mode, momentum, channel_dim, eps
        self.register_buffer("scale", torch.empty(0))
        self.num_batches_tracked = 0

    def forward(self, x):
        if x.dim() < 2:
            raise ValueError("Channel-wise rate calibration requires activation tensors with at least 2 dimensions.")
        d = self.channel_dim + x.dim() if self.channel_dim < 0 else self.channel_dim
        if not 0 <= d < x.dim():
            raise ValueError("channel_dim is out of range.")
        stat = torch.clamp(x.detach(), min=0)
        stat = stat.float() if stat.dtype in (torch.float16, torch.bfloat16) else stat
        rows = stat.movedim(d, 0).reshape(stat.shape[d], -1)
        try:
            s_t = _scale_statistic(rows, self.mode, reduce_dim=1)
        except (ValueError, RuntimeError) as exc:
            raise NotImplementedError(_BAD_MODE) from exc
        s_t = torch.clamp(s_t.to(device=x.device, dtype=x.dtype), min=self.eps)
        self.scale = (s_t if self.num_batches_tracked == 0 else (1 - self.momentum) * self.scale.to(s_t) + self.momentum * s_t).detach()
        self.num_batches_tracked += x.shape[0]
        return x

    def compute_threshold(self) -> torch.Tensor:
        if self.scale.numel() == 0:
            raise ValueError("No calibration activations have been recorded.")
        if not torch.isfinite(self.scale).all() or (self.scale <= 0).any():
            raise ValueError("Channel-wise thresholds must be finite positive values.")
        return self.scale.detach()


class RateCodingRecipe(ConversionRecipe):
    """``dataloader`` yields calibration batches; ``mode``: ``"Max"``, ``"99.9%"`` or a float in (0, 1];
    ``fuse_flag``: fold BatchNorm first; ``channel_wise``: one threshold per channel (``pre_spike_maxpool``
    moves a following MaxPool2d before the neuron, ``half_threshold`` starts neurons at half threshold)."""

    def __init__(self, dataloader: Iterable, mode: Union[str, float] = "Max", momentum: float = 0.1, fuse_flag: bool = True,
                 channel_wise: bool = False, channel_dim: int = 1, pre_spike_maxpool: bool = False, half_threshold: bool = False,
                 eps: float = 1e-6, neuron_factory: Optional[NeuronFactory] = None) -> None:
        self.dataloader, self.mode, self.momentum, self.fuse_flag = dataloader, mode, momentum, fuse_flag
        self.channel_wise, self.channel_dim, self.pre_spike_maxpool, self.half_threshold, self.eps = \
            channel_wise, channel_dim, pre_spike_maxpool, half_threshold, eps
        if channel_wise and half_threshold and neuron_factory is not None:
            raise ValueError("RateCodingRecipe(channel_wise=True, half_threshold=True) does not support custom neuron_factory.")
        self.neuron_factory = neuron_factory if neuron_factory is not None else NeuronFactory()

    def validate(self, converter) -> None:
        if self.dataloader is None:
            raise ValueError("RateCodingRecipe requires a dataloader. Pass dataloader to RateCodingRecipe.")
        validate_rate_coding_mode(self.mode)
        m = self.momentum
        if not isinstance(m, (int, float)) or isinstance(m, bool) or not math.isfinite(float(m)) or not 0.0 <= m <= 1.0:
            raise ValueError("momentum must be a finite number in [0, 1].")
        for name in ("channel_wise", "pre_spike_maxpool", "half_threshold"):
            if not isinstance(getattr(self, name), bool):
                raise ValueError(f"{name} must be bool.")
        if not isinstance(self.channel_dim, int):
            raise ValueError("channel_dim must be int.")
        if not (isinstance(self.eps, (int, float)) and self.eps > 0):
            raise ValueError("eps must be a positive number.")

    def before_trace(self, converter, ann):
        ann.eval()
        return ann

    def after_trace(self, converter, fx_model):
        return _fuse_conv_bn(fx_model, self.fuse_flag).to(converter.device)

    def insert_observers(self, converter, fx_model):
        counts: Dict[str, int] = {}
        modules = dict(fx_model.named_modules())
        for node in list(fx_model.graph.nodes):
            if not _is_relu(node, modules):
                continue
            parent = node.target.rpartition(".")[0]
            i = counts.get(parent, 0)
            counts[parent] = i + 1
            leaf, hook = self._new_hook(i)
            hook.train()
            source = node
            users = list(node.users)
            if self.channel_wise and self.pre_spike_maxpool and len(users) == 1 and users[0].op == "call_module" \
                    and isinstance(modules.get(users[0].target), nn.MaxPool2d):
                source = users[0]
            hook_node = _insert(fx_model, f"{parent}.{leaf}" if parent else leaf, source, hook, (source,))
            if self.channel_wise:
                for u in list(source.users):
                    if u is not hook_node:
                        u.replace_input_with(source, hook_node)
        fx_model.graph.lint()
        fx_model.recompile()
        return fx_model.to(converter.device)

    _channel_hook_type = None          # set below (class attribute of the hook used by the channel-wise path)
    _channel_leaf = "channel_voltage_hook_"

    def _new_hook(self, index: int):
        if self.channel_wise:
            return f"{self._channel_leaf}{index}", ChannelVoltageHook(self.mode, self.momentum, self.channel_dim, self.eps)
        return f"voltage_hook_{index}", VoltageHook(momentum=self.momentum, mode=self.mode)

    def calibrate(self, converter, fx_model):
        with torch.no_grad():
            for data in self.dataloader:
                x = _extract_batch_input(data)
                if isinstance(x, (list, tuple, dict)):
                    raise ValueError("RateCodingRecipe supports single-input calibration batches only. For multi-input models, "
                                     "subclass ConversionRecipe or RateCodingRecipe and override calibrate().")
                fx_model(x.to(converter.device) if isinstance(x, torch.Tensor) else torch.as_tensor(x, device=converter.device))
        return fx_model

    def replace(self, converter, fx_model):
        modules = dict(fx_model.named_modules())
        for hook_node in list(fx_model.graph.nodes):
            if hook_node.op != "call_module" or not hook_node.args or not isinstance(hook_node.args[0], fx.Node):
                continue
            hook, src = modules.get(hook_node.target), hook_node.args[0]
            if self.channel_wise and isinstance(hook, self._channel_hook_type or ChannelVoltageHook):
                act = src
                if not _is_relu(act, modules):
                    if not isinstance(modules.get(src.target), nn.MaxPool2d) or not src.args or not isinstance(src.args[0], fx.Node) \
                            or not _is_relu(src.args[0], modules):
                        continue
                    act = src.args[0]
                self._replace_channelwise(fx_model, act, hook_node, hook)
            elif not self.channel_wise and isinstance(hook, VoltageHook) and _is_relu(src, modules):
                self._replace_layerwise(fx_model, src, hook_node, hook)
        fx_model.graph.lint()
        fx_model.delete_all_unused_submodules()
        fx_model.recompile()
        return adapt_step_mode_graph(fx_model, context="RateCodingRecipe step-mode backend").to(converter.device)

    def _scalar_threshold(self, sn) -> float:
        th = getattr(sn, "v_threshold", 1.0)
        if hasattr(th, "item") and (not hasattr(th, "numel") or th.numel() == 1):
            th = th.item()
        return th

    def _replace_layerwise(self, fx_model, act, hook_node, hook):
        scale = float(hook.scale.item())
        if not scale > 0.0 or not math.isfinite(scale):
            raise ValueError(f"Threshold must be a finite positive number, got {scale} for hook {hook_node.target!r}.")
        parent, _, leaf = hook_node.target.rpartition(".")
        prefix = ".".join(filter(None, [parent, leaf.replace("voltage_hook_", "spiking_")]))
        sn = self.neuron_factory.create(scale=scale)
        n0 = _insert(fx_model, f"{prefix}.scaler0", hook_node, VoltageScaler(self._scalar_threshold(sn) / scale), act.args)
        n1 = _insert(fx_model, f"{prefix}.if_node", n0, sn, (n0,))
        n2 = _insert(fx_model, f"{prefix}.scaler1", n1, VoltageScaler(scale), (n1,))
        hook_node.replace_all_uses_with(n2)
        act.replace_all_uses_with(n2)
        fx_model.graph.erase_node(hook_node)
        fx_model.graph.erase_node(act)

    def _replace_channelwise(self, fx_model, act, hook_node, hook):
        src = hook_node.args[0]
        pooled_first = src is not act
        if pooled_first:
            src.replace_input_with(act, act.args[0])
        threshold = hook.compute_threshold()
        parent, _, leaf = hook_node.target.rpartition(".")
        prefix = ".".join(filter(None, [parent, leaf.replace(self._channel_leaf, self._channel_leaf.replace("voltage_hook_", "spiking_").replace("hook_", "spiking_"))]))
        if self.half_threshold:
            sn, th = neuron.HalfThresholdIFNode(), 1.0
        else:
            sn = self.neuron_factory.create(scale=1.0)
            th = self._scalar_threshold(sn)
            if not isinstance(th, (int, float)):
                raise ValueError("Channel-wise RateCodingRecipe requires a scalar neuron threshold.")
            if not th > 0.0 or not math.isfinite(th):
                raise ValueError(f"Channel-wise RateCodingRecipe requires a finite positive neuron threshold, got {th}.")
        n0 = _insert(fx_model, f"{prefix}.scaler0", hook_node, ChannelVoltageScaler(th / threshold, channel_dim=self.channel_dim),
                     (src,) if pooled_first else act.args)
        n1 = _insert(fx_model, f"{prefix}.if_node", n0, sn, (n0,))
        n2 = _insert(fx_model, f"{prefix}.scaler1", n1, ChannelVoltageScaler(threshold, channel_dim=self.channel_dim), (n1,))
        hook_node.replace_all_uses_with(n2)
        fx_model.graph.erase_node(hook_node)
        if not pooled_first:
            act.replace_all_uses_with(n2)
        fx_model.graph.erase_node(act)
