"""Exact conversion of transformer-style networks: every supported module becomes its
temporal-difference operator; the sum of the converted network's outputs over ``T`` steps equals the
ANN's output on the sum of the inputs, for any ``T``.
Parity: ``spikingjelly/activation_based/ann2snn/recipes/transformer_td_equivalent.py:1-530``."""
from __future__ import annotations

import operator

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import fx

from ... import base

from ..operators import (SNNElementWiseProduct, SNNMatrixOperator, TDGELU, TDModule, TDSiLU, TDSoftmax, _td_module_from_ann)
from .base import FXConversionRecipe
from .step_mode_adapters import adapt_step_mode_graph, lift_tensor_functions

__all__ = ["TransformerTDEquivalentRecipe"]

_LINEAR_SAFE = (nn.Dropout, nn.Identity, nn.Flatten)
#: placeholder names that carry no time axis in multi-step mode
STATIC_INPUT_NAMES = frozenset({"attention_mask", "attn_mask", "causal_mask", "decoder_attention_mask", "encoder_attention_mask",
                                "key_padding_mask", "mask", "padding_mask"})
_METHOD_MODULES = {"softmax": lambda node: TDSoftmax(node.kwargs.get("dim", node.args[1] if len(node.args) > 1 else -1)),
                   "matmul": lambda node: SNNMatrixOperator()}
_FUNCTION_MODULES = {F.gelu: lambda node: TDGELU(node.kwargs.get("approximate", "none")), F.silu: lambda node: TDSiLU(),
                     torch.nn.functional.softmax: lambda node: TDSoftmax(node.kwargs.get("dim", node.args[1] if len(node.args) > 1 else -1)),
                     torch.softmax: lambda node: TDSoftmax(node.kwargs.get("dim", node.args[1] if len(node.args) > 1 else -1))}


class TransformerTDEquivalentRecipe(FXConversionRecipe):
    """``time_steps``: optional number of steps the converted model is meant to run (recorded on it as ``time_steps``; the
    operators themselves work for any length).  ``step_mode``: mode given to the created operators.  Unsupported non-linear
    modules raise (``strict=True``, default) or are left untouched (which breaks exactness)."""

    def __init__(self, time_steps: Optional[int] = None, step_mode: str = "m", strict: bool = True) -> None:
        self.time_steps, self.step_mode, self.strict = time_steps, step_mode, strict

    def validate(self, converter) -> None:
        t = self.time_steps
        if t is not None and (not isinstance(t, int) or isinstance(t, bool) or t <= 0):
            raise ValueError("time_steps must be a positive integer when set.")

    def before_trace(self, converter, ann):
        ann.eval()
        return ann

    def _operator_for(self, node: fx.Node):
        """``(operator module, its inputs)`` for a function or method node that has a temporal-difference form, else None."""
        is_node = lambda *xs: all(isinstance(x, fx.Node) for x in xs)
        if node.op == "call_function":
            if node.target in _FUNCTION_MODULES and is_node(node.args[0]):
                return _FUNCTION_MODULES[node.target](node), (node.args[0],)
            if node.target in (torch.matmul, operator.matmul) and len(node.args) >= 2 and is_node(*node.args[:2]):
                return SNNMatrixOperator(), tuple(node.args[:2])
            if node.target in (operator.mul, torch.mul) and len(node.args) >= 2 and is_node(*node.args[:2]):
                return SNNElementWiseProduct(), tuple(node.args[:2])
        elif node.op == "call_method" and node.target in _METHOD_MODULES and node.args and is_node(node.args[0]):
            if node.target == "matmul":
                return (SNNMatrixOperator(), tuple(node.args[:2])) if len(node.args) >= 2 and is_node(node.args[1]) else None
            return _METHOD_MODULES[node.target](node), (node.args[0],)
        return None

    def replace(self, converter, fx_model: fx.GraphModule) -> fx.GraphModule:
        modules = dict(fx_model.named_modules())
        n_new = 0
        for node in list(fx_model.graph.nodes):
            if node.op == "call_module":
                m = modules.get(node.target)
                if isinstance(m, (TDModule, base.MemoryModule)) or isinstance(m, _LINEAR_SAFE):
                    continue
                td = _td_module_from_ann(m, self.step_mode)
                if td is None:
                    if self.strict:
                        raise NotImplementedError(f"TransformerTDEquivalentRecipe has no temporal-difference operator for "
                                                  f"{type(m).__name__} at '{node.target}'.")
                    continue
                parent, _, child = node.target.rpartition(".")
                setattr(fx_model.get_submodule(parent) if parent else fx_model, child, td)
                continue
            found = self._operator_for(node)
            if found is None:
                continue
            new, args = found
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
        # what is left (stateless layers, tensor functions) follows the step mode of the network
        adapt_step_mode_graph(fx_model, context=type(self).__name__)
        static = [n.target for n in fx_model.graph.nodes if n.op == "placeholder" and n.target in STATIC_INPUT_NAMES]
        return lift_tensor_functions(fx_model, static_inputs=static)
