"""What a conversion recipe is (``spikingjelly/activation_based/ann2snn/recipes/base.py:22-492``).

An FX recipe works on a traced ``GraphModule`` and is asked, in the order of :data:`FX_STAGES`, to validate its settings,
touch the model before and after tracing, insert observers, calibrate, replace nodes and finalise.  A module recipe gets
the module tree itself.  Every stage is optional: a recipe overrides the ones it needs, the rest pass their argument
through."""
from __future__ import annotations

import torch.nn as nn
from torch import fx

__all__ = ["ConversionRecipe", "FXConversionRecipe", "ModuleConversionRecipe", "replace_submodule", "FX_STAGES"]

#: graph stages in execution order (``validate`` and ``before_trace`` come before there is a graph)
FX_STAGES = ("after_trace", "insert_observers", "calibrate", "replace", "finalize")


def replace_submodule(fx_model: fx.GraphModule, target: str, module: nn.Module) -> None:
    """``fx_model.<target> = module`` for a dotted ``target``."""
    *owner_path, leaf = target.split(".")
    owner = fx_model.get_submodule(".".join(owner_path)) if owner_path else fx_model
    setattr(owner, leaf, module)


class FXConversionRecipe:
    """Base of the graph recipes.  ``converter`` is the running converter (``converter.device`` is where the result goes).
    Every stage returns what it was given unless a recipe overrides it."""

    def validate(self, converter) -> None:
        """Check the recipe's own settings; raise on a contradiction."""

    def before_trace(self, converter, ann: nn.Module) -> nn.Module:
        """Prepare the ANN for tracing, e.g. switch to eval mode."""
        return ann

    def after_trace(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        """Clean the traced graph, e.g. fold batch norms."""
        return fx_model

    def insert_observers(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        return fx_model

    def calibrate(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        """Run the calibration data through the observed graph."""
        return fx_model

    def replace(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        """Put the spiking modules in."""
        return fx_model

    def finalize(self, converter, fx_model: fx.GraphModule) -> nn.Module:
        return fx_model

    def run_graph_stages(self, converter, graph: fx.GraphModule) -> nn.Module:
        """All stages that take the traced graph, in order."""
        for stage in FX_STAGES:
            graph = getattr(self, stage)(converter, graph)
        return graph


#: historical name of the graph recipe base
ConversionRecipe = FXConversionRecipe


class ModuleConversionRecipe:
    """Base of the recipes that rewrite modules in place, without tracing."""

    def validate(self, converter) -> None:
        """Check the recipe's own settings; raise on a contradiction."""

    def convert_module(self, converter, ann: nn.Module) -> nn.Module:
        """The converted module; the base class returns ``ann`` unchanged."""
        return ann
