"""Recipe protocol of the converters.  An FX recipe transforms a traced ``GraphModule`` in stages
(validate, before_trace, after_trace, insert_observers, calibrate, replace, finalize); a module recipe
rewrites the module tree directly.  Parity: ``spikingjelly/activation_based/ann2snn/recipes/base.py:15-492``."""
from __future__ import annotations

import torch.nn as nn
from torch import fx

__all__ = ["ConversionRecipe", "FXConversionRecipe", "ModuleConversionRecipe", "replace_submodule"]


def replace_submodule(fx_model: fx.GraphModule, target: str, module: nn.Module) -> None:
    parent_name, _, child = target.rpartition(".")
    setattr(fx_model.get_submodule(parent_name) if parent_name else fx_model, child, module)


class FXConversionRecipe:
    """Every stage defaults to the identity; ``converter`` gives access to ``converter.device``."""

    def validate(self, converter) -> None:
        return None

    def before_trace(self, converter, ann: nn.Module) -> nn.Module:
        return ann

    def after_trace(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        return fx_model

    def insert_observers(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        return fx_model

    def calibrate(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        return fx_model

    def replace(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        return fx_model

    def finalize(self, converter, fx_model: fx.GraphModule) -> nn.Module:
        return fx_model


ConversionRecipe = FXConversionRecipe


class ModuleConversionRecipe:
    def validate(self, converter) -> None:
        return None

    def convert_module(self, converter, ann: nn.Module) -> nn.Module:
        return ann
