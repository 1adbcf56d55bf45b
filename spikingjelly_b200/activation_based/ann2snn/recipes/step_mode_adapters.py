"""After conversion the graph holds plain ``torch.nn`` layers and tensor functions next to stateful step-mode modules.
Two passes make ``functional.set_step_mode(snn, "m")`` turn the whole converted network into one that consumes
``[T, B, ...]`` sequences (parity: ``spikingjelly/activation_based/ann2snn/recipes/step_mode_adapters.py:15-636``):

* :func:`adapt_step_mode_graph` swaps every stateless layer for its step-mode twin (same parameters, same state-dict
  keys);
* :func:`lift_tensor_functions` wraps every tensor function or method of the graph that touches the time-varying signal
  (``cat``, ``reshape``, ``transpose``, ``x[:, 0]``, ``x.shape`` ...) in a :class:`StepFunction`.  In single-step mode
  the wrapper is the function itself; in multi-step mode it maps the function over the leading time axis with
  ``torch.vmap``, so every ``dim=`` argument, slice and shape query keeps the meaning it had in the traced per-step
  program, whatever the operator.  (The reference rewrites a fixed list of operators one by one, shifting their
  dimension arguments; mapping over time needs no list.)  Which inputs vary in time is decided once, from the graph:
  placeholders and outputs of stateful modules do, attributes (masks, index buffers) do not."""
from __future__ import annotations

import builtins
import copy
import operator
from typing import Any, Callable, Iterable, Sequence, Set, Tuple, Type, Union

import torch
import torch.nn as nn
from torch import fx
from torch.utils import _pytree as pytree

from ... import base, layer

__all__ = ["adapt_step_mode_graph", "lift_tensor_functions", "StepFunction", "STEP_MODULE_TYPES"]

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


def adapt_step_mode_graph(fx_model: fx.GraphModule, context: str = "step-mode backend", wrap_module_types=(), safe_module_types=(),
                          safe_call_functions=()) -> fx.GraphModule:
    """Replace, in place, every ``call_module`` target whose type is in ``wrap_module_types`` by its step-mode twin.  With no
    types given, the stateless layers a rate-coded network is made of are wrapped (``_RATE_CODING_STATELESS_MODULE_TYPES``)."""
    wrap_module_types = tuple(wrap_module_types) or _RATE_CODING_STATELESS_MODULE_TYPES
    safe_module_types = tuple(safe_module_types) or _RATE_CODING_SAFE_MODULE_TYPES
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


# ---------------------------------------------------------------------------------------------------------------------
# tensor functions over the time axis
# ---------------------------------------------------------------------------------------------------------------------
_SHAPE_QUERIES = frozenset({"size", "dim", "numel", "ndimension", "shape", "dtype", "device", "is_floating_point"})


class StepFunction(nn.Module, base.StepModule):
    """One tensor function (``target`` is a callable) or tensor method (``target`` is its name) of a traced program.
    ``temporal`` holds the positions, among the flattened ``(args, kwargs)`` leaves, of the inputs that carry a leading
    time axis in multi-step mode; the others are passed unchanged to every step."""

    def __init__(self, target: Union[str, Callable], temporal: Sequence[int], step_mode: str = "s") -> None:
        super().__init__()
        self.target, self.temporal, self.step_mode = target, tuple(temporal), step_mode

    def _call(self, *args, **kwargs):
        if isinstance(self.target, str):
            return getattr(args[0], self.target)(*args[1:], **kwargs)
        return self.target(*args, **kwargs)

    def _is_shape_query(self) -> bool:
        if isinstance(self.target, str):
            return self.target in _SHAPE_QUERIES
        return self.target is builtins.getattr

    def forward(self, *args, **kwargs):
        if self.step_mode == "s":
            return self._call(*args, **kwargs)
        leaves, spec = pytree.tree_flatten((args, kwargs))
        moving = [i for i in self.temporal if i < len(leaves) and torch.is_tensor(leaves[i])]
        if not moving:
            return self._call(*args, **kwargs)
        if self._is_shape_query() or (self.target is builtins.getattr):
            first = list(leaves)
            for i in moving:
                first[i] = leaves[i][0]                      # every step has the same shape: ask the first one
            a, k = pytree.tree_unflatten(first, spec)
            return self._call(*a, **k)
        in_dims = tuple(0 if i in moving else None for i in range(len(leaves)))

        def per_step(*step_leaves):
            a, k = pytree.tree_unflatten(list(step_leaves), spec)
            return self._call(*a, **k)
        return torch.vmap(per_step, in_dims=in_dims)(*leaves)

    def extra_repr(self) -> str:
        name = self.target if isinstance(self.target, str) else getattr(self.target, "__name__", repr(self.target))
        return f"{name}, temporal={list(self.temporal)}, step_mode={self.step_mode}"


def _temporal_nodes(fx_model: fx.GraphModule, static_inputs: Iterable[str]) -> Set[fx.Node]:
    """Nodes whose value changes from step to step: placeholders (but the named static ones), calls of stateful modules,
    and everything computed from one of those."""
    static_inputs = set(static_inputs)
    modules = dict(fx_model.named_modules())
    moving: Set[fx.Node] = set()
    for node in fx_model.graph.nodes:
        if node.op == "placeholder":
            if node.target not in static_inputs:
                moving.add(node)
        elif node.op == "call_module" and isinstance(modules.get(node.target), base.MemoryModule):
            moving.add(node)
        elif node.op in ("call_module", "call_function", "call_method") and any(n in moving for n in node.all_input_nodes):
            moving.add(node)
    return moving


def lift_tensor_functions(fx_model: fx.GraphModule, *, static_inputs: Iterable[str] = (), keep: Iterable[Callable] = ()) -> fx.GraphModule:
    """Replace, in place, every ``call_function`` / ``call_method`` node with a time-varying input by a
    :class:`StepFunction` module call.  ``static_inputs``: placeholder names that never carry a time axis (masks);
    ``keep``: functions to leave alone (element-wise ones that mean the same with and without a time axis need no
    wrapper, but wrapping them is harmless)."""
    moving = _temporal_nodes(fx_model, static_inputs)
    keep = set(keep)
    taken = set(dict(fx_model.named_modules()))
    n = 0
    for node in list(fx_model.graph.nodes):
        if node.op not in ("call_function", "call_method") or node not in moving or node.target in keep:
            continue
        if node.op == "call_function" and node.target is operator.getitem and node.args[0] not in moving:
            continue
        leaves, _ = pytree.tree_flatten((tuple(node.args), dict(node.kwargs)))
        temporal = [i for i, leaf in enumerate(leaves) if isinstance(leaf, fx.Node) and leaf in moving]
        # indexing the tuple a module returned (attention output and weights) is not a tensor operation
        if node.target is operator.getitem and isinstance(node.args[1], int) and _returns_tuple(node.args[0], fx_model):
            continue
        while f"step_function_{n}" in taken:
            n += 1
        target = f"step_function_{n}"
        taken.add(target)
        fx_model.add_submodule(target, StepFunction(node.target, temporal, step_mode="s"))
        with fx_model.graph.inserting_after(node):
            call = fx_model.graph.call_module(target, args=tuple(node.args), kwargs=dict(node.kwargs))
        node.replace_all_uses_with(call)
        fx_model.graph.erase_node(node)
        moving.add(call)
    fx_model.graph.lint()
    fx_model.recompile()
    return fx_model


def _returns_tuple(node: Any, fx_model: fx.GraphModule) -> bool:
    if not isinstance(node, fx.Node) or node.op != "call_module":
        return False
    from ..operators import TDMultiheadAttention
    return isinstance(fx_model.get_submodule(node.target), (nn.MultiheadAttention, TDMultiheadAttention))
