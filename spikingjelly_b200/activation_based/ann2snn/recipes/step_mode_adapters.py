"""After conversion the graph holds plain ``torch.nn`` layers next to spiking neurons.  This pass
swaps every stateless layer for its step-mode twin (same parameters, same state-dict keys) so that
``functional.set_step_mode(snn, "m")`` makes the whole converted network consume ``[T, B, ...]`` sequences.
Parity: ``spikingjelly/activation_based/ann2snn/recipes/step_mode_adapters.py:15-636``."""
from __future__ import annotations

import copy
from typing import Tuple, Type

import torch.nn as nn
from torch import fx

from ... import layer

__all__ = ["adapt_step_mode_graph", "STEP_MODULE_TYPES"]

STEP_MODULE_TYPES: Tuple[Tuple[Type[nn.Module], Type[nn.Module]], ...] = (
    (nn.Conv1d, layer.Conv1d), (nn.Conv2d, layer.Conv2d), (nn.Conv3d, layer.Conv3d),
    (nn.ConvTranspose1d, layer.ConvTranspose1d), (nn.ConvTranspose2d, layer.ConvTranspose2d), (nn.ConvTranspose3d, layer.ConvTranspose3d),
    (nn.Linear, layer.Linear), (nn.MaxPool1d, layer.MaxPool1d), (nn.MaxPool2d, layer.MaxPool2d), (nn.MaxPool3d, layer.MaxPool3d),
    (nn.AvgPool1d, layer.AvgPool1d), (nn.AvgPool2d, layer.AvgPool2d), (nn.AvgPool3d, layer.AvgPool3d),
    (nn.AdaptiveAvgPool1d, layer.AdaptiveAvgPool1d), (nn.AdaptiveAvgPool2d, layer.AdaptiveAvgPool2d),
    (nn.AdaptiveAvgPool3d, layer.AdaptiveAvgPool3d), (nn.BatchNorm1d, layer.BatchNorm1d), (nn.BatchNorm2d, layer.BatchNorm2d),
    (nn.BatchNorm3d, layer.BatchNorm3d), (nn.GroupNorm, layer.GroupNorm), (nn.Upsample, layer.Upsample), (nn.Flatten, layer.Flatten),
    (nn.Dropout, layer.Dropout), (nn.Dropout2d, layer.Dropout2d))
_RATE_CODING_STATELESS_MODULE_TYPES = tuple(s for s, _ in STEP_MODULE_TYPES)
_RATE_CODING_SAFE_MODULE_TYPES = (nn.ReLU,)


def _make_step_module(module: nn.Module) -> nn.Module:
    if isinstance(module, (nn.MaxPool1d, nn.MaxPool2d, nn.MaxPool3d)) and module.return_indices:
        raise ValueError("Step-mode adapter does not support return_indices=True.")
    if isinstance(module, (nn.Dropout, nn.Dropout2d)):
        if module.inplace:
            raise ValueError(f"Step-mode adapter does not support {type(module).__name__} with inplace=True.")
        return (layer.Dropout2d if isinstance(module, nn.Dropout2d) else layer.Dropout)(p=module.p).train(module.training)
    for src, dst in STEP_MODULE_TYPES:
        if type(module) is dst:
            return module
        if isinstance(module, src):
            twin = copy.deepcopy(module)
            twin.__class__ = dst               # the step-mode class extends the torch class: parameters and keys are unchanged
            twin.step_mode = "s"
            return twin
    raise TypeError(type(module).__name__)


def adapt_step_mode_graph(fx_model: fx.GraphModule, *, context: str = "step-mode backend", wrap_module_types=_RATE_CODING_STATELESS_MODULE_TYPES,
                          safe_module_types=_RATE_CODING_SAFE_MODULE_TYPES, safe_call_functions=()) -> fx.GraphModule:
    """Replace, in place, every ``call_module`` target whose type is in ``wrap_module_types`` by its
    step-mode twin."""
    modules = dict(fx_model.named_modules())
    seen = {}
    for node in fx_model.graph.nodes:
        if node.op != "call_module" or node.target not in modules:
            continue
        m = modules[node.target]
        if isinstance(m, tuple(wrap_module_types)) and not hasattr(m, "step_mode"):
            if id(m) not in seen:
                seen[id(m)] = _make_step_module(m)
            parent, _, child = node.target.rpartition(".")
            setattr(fx_model.get_submodule(parent) if parent else fx_model, child, seen[id(m)])
    fx_model.recompile()
    return fx_model
