"""Converters: drive a recipe over a model.  ``FXConverter`` (alias ``Converter``) traces the ANN with
``torch.fx`` and hands the graph to an ``FXConversionRecipe``; ``ModuleConverter`` hands the module tree to
a ``ModuleConversionRecipe``.  Both run under ``no_grad``, restore every module's training flag and
return the converted network on the requested device.
Parity: ``spikingjelly/activation_based/ann2snn/converter.py:23-355``."""
from __future__ import annotations

import logging
import threading
import time
import types
import warnings
from typing import Optional, Union

import torch
import torch.nn as nn
from torch import fx

from ...logger import logger
from .recipes import FXConversionRecipe, ModuleConversionRecipe, TransformerTDEquivalentRecipe

__all__ = ["Converter", "FXConverter", "ModuleConverter"]

_TRACE_LOCK = threading.RLock()


def _resolve_device(ann: nn.Module, configured) -> torch.device:
    if configured is not None:
        return torch.device(configured)
    p = next(ann.parameters(), None)
    return p.device if p is not None else torch.device("cpu")


def _symbolic_trace(root: nn.Module) -> fx.GraphModule:
    with _TRACE_LOCK:
        tracer = fx.Tracer()
        graph = tracer.trace(root)
    for node in graph.nodes:                       # PEP 604 unions in annotations confuse FX code generation
        if isinstance(node.type, types.UnionType):
            node.type = None
    return fx.GraphModule(tracer.root, graph)


class _ConverterBase:
    def _run(self, ann: nn.Module, body):
        configured = self.device
        flags = {m: m.training for m in ann.modules()}
        t0 = time.perf_counter()
        try:
            self.device = _resolve_device(ann, configured)
            with torch.no_grad():
                self.recipe.validate(self)
                out = body(ann)
            if logger.isEnabledFor(logging.INFO):
                logger.info("ann2snn_conversion_summary converter=%s recipe=%s device=%s modules=%s elapsed_ms=%.3f", type(self).__name__,
                            type(self.recipe).__name__, self.device, sum(1 for _ in out.modules()), (time.perf_counter() - t0) * 1e3)
            return out
        finally:
            for m, flag in flags.items():
                m.training = flag
            self.device = configured


class FXConverter(_ConverterBase):
    """``recipe``: an ``FXConversionRecipe`` or the name ``"transformer_td_equivalent"``."""

    def __init__(self, recipe: Union[str, FXConversionRecipe], device: Optional[Union[torch.device, str]] = None) -> None:
        self.recipe = self._resolve_recipe(recipe)
        self.device = device

    @staticmethod
    def _resolve_recipe(recipe):
        if isinstance(recipe, FXConversionRecipe):
            return recipe
        if isinstance(recipe, ModuleConversionRecipe):
            raise TypeError("FXConverter/Converter requires an FXConversionRecipe. Use ModuleConverter for ModuleConversionRecipe instances.")
        if recipe == "transformer_spike_equivalent":
            warnings.warn("The 'transformer_spike_equivalent' recipe string is deprecated; use 'transformer_td_equivalent' instead.",
                          DeprecationWarning, stacklevel=3)
            return TransformerTDEquivalentRecipe()
        if recipe == "transformer_td_equivalent":
            return TransformerTDEquivalentRecipe()
        if recipe == "rate_coding":
            raise ValueError("The rate_coding recipe requires parameters. Pass RateCodingRecipe(dataloader=...) to Converter.")
        if recipe == "sta_transformer":
            raise ValueError("The sta_transformer recipe requires parameters. Pass STATransformerRecipe(dataloader=..., time_steps=...) to Converter.")
        if isinstance(recipe, str):
            raise ValueError(f"Unknown ann2snn conversion recipe: {recipe!r}.")
        raise TypeError(f"recipe must be a recipe name string or an FXConversionRecipe instance, but got {type(recipe).__name__}.")

    def convert(self, ann: nn.Module) -> nn.Module:
        def body(ann):
            r = self.recipe
            model = _symbolic_trace(r.before_trace(self, ann)).to(self.device)
            for stage in (r.after_trace, r.insert_observers, r.calibrate, r.replace, r.finalize):
                model = stage(self, model)
            return model
        return self._run(ann, body)


class ModuleConverter(_ConverterBase):
    def __init__(self, recipe: ModuleConversionRecipe, device: Optional[Union[torch.device, str]] = None) -> None:
        if isinstance(recipe, FXConversionRecipe):
            raise TypeError("ModuleConverter requires a ModuleConversionRecipe. Use FXConverter/Converter for FXConversionRecipe instances.")
        if not isinstance(recipe, ModuleConversionRecipe):
            raise TypeError(f"recipe must be a ModuleConversionRecipe instance, but got {type(recipe).__name__}.")
        self.recipe, self.device = recipe, device

    def convert(self, ann: nn.Module) -> nn.Module:
        def body(ann):
            out = self.recipe.convert_module(self, ann)
            if not isinstance(out, nn.Module):
                raise TypeError(f"ModuleConversionRecipe.convert_module must return a torch.nn.Module, got {type(out).__name__}.")
            return out.to(self.device)
        return self._run(ann, body)


Converter = FXConverter
