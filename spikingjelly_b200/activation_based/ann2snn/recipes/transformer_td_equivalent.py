"""Exact conversion of transformer-style networks: every supported module becomes its
temporal-difference operator; the sum of the converted network's outputs over ``T`` steps equals the
ANN's output on the sum of the inputs, for any ``T``.
Parity: ``spikingjelly/activation_based/ann2snn/recipes/transformer_td_equivalent.py:1-530``."""
from __future__ import annotations

import operator

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import fx

from ..operators import (SNNElementWiseProduct, SNNMatrixOperator, TDGELU, TDModule, TDSiLU, TDSoftmax, _td_module_from_ann)
from .base import FXConversionRecipe

__all__ = ["TransformerTDEquivalentRecipe"]

_LINEAR_SAFE = (nn.Dropout, nn.Identity, nn.Flatten)
_FUNCTION_MODULES = {F.gelu: lambda node: TDGELU(node.kwargs.get("approximate", "none")), F.silu: lambda node: TDSiLU(),
                     torch.nn.functional.softmax: lambda node: TDSoftmax(node.kwargs.get("dim", node.args[1] if len(node.args) > 1 else -1)),
                     torch.softmax: lambda node: TDSoftmax(node.kwargs.get("dim", node.args[1] if len(node.args) > 1 else -1))}


class TransformerTDEquivalentRecipe(FXConversionRecipe):
    """``step_mode``: mode given to the created operators.  Unsupported non-linear modules raise
    (``strict=True``, default) or are left untouched (which breaks exactness)."""

    def __init__(self, step_mode: str = "m", strict: bool = True) -> None:
        self.step_mode, self.strict = step_mode, strict

    def before_trace(self, converter, ann):
        ann.eval()
        return ann

    def replace(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        modules = dict(fx_model.named_modules())
        n_new = 0
        for node in list(fx_model.graph.nodes):
            if node.op == "call_module":
                m = modules.get(node.target)
                if isinstance(m, TDModule) or isinstance(m, _LINEAR_SAFE):
                    continue
                td = _td_module_from_ann(m, self.step_mode)
                if td is None:
                    if self.strict:
                        raise NotImplementedError(f"TransformerTDEquivalentRecipe has no temporal-difference operator for "
                                                  f"{type(m).__name__} at '{node.target}'.")
                    continue
                parent, _, child = node.target.rpartition(".")
                setattr(fx_model.get_submodule(parent) if parent else fx_model, child, td)
            elif node.op == "call_function":
                new = None
                if node.target in _FUNCTION_MODULES:
                    new, args = _FUNCTION_MODULES[node.target](node), (node.args[0],)
                elif node.target in (torch.matmul, operator.matmul) and all(isinstance(a, fx.Node) for a in node.args[:2]):
                    new, args = SNNMatrixOperator(), tuple(node.args[:2])
                elif node.target in (operator.mul, torch.mul) and all(isinstance(a, fx.Node) for a in node.args[:2]):
                    new, args = SNNElementWiseProduct(), tuple(node.args[:2])
                if new is None:
                    continue
                new.step_mode = self.step_mode
                target = f"td_function_{n_new}"
                n_new += 1
                fx_model.add_submodule(target, new)
                with fx_model.graph.inserting_after(node):
                    repl = fx_model.graph.call_module(target, args=args)
                node.replace_all_uses_with(repl)
                fx_model.graph.erase_node(node)
        fx_model.graph.lint()
        fx_model.recompile()
        return fx_model
