"""Operation counting by dispatch interception.

``DispatchCounterMode([counters])`` is a context manager that sees every ATen call (forward, backward
and optimizer), evaluates each counter's rule for the called operator and books the value under
every module that is active at that moment (``"Global"`` always is).  ``FunctionCounterMode`` does the
same at the ``torch.*`` function level.  A rule is ``rule(args, kwargs, out) -> int``.

The native kernels of this package are ATen-level custom operators (``torch.ops.sjb200.*``), so they
appear in the stream like any other operator; counters ship rules for them next to the ATen rules.

Parity: ``spikingjelly/activation_based/op_counter/base.py:17-801``.
"""
from __future__ import annotations

import logging
from collections import defaultdict
from typing import Any, Callable, Dict, List, Optional, Set

import torch
import torch.nn as nn
from torch.autograd.graph import register_multi_grad_hook
from torch.overrides import TorchFunctionMode, resolve_name
from torch.utils._python_dispatch import TorchDispatchMode
from torch.utils._pytree import tree_flatten
from torch.utils.module_tracker import ModuleTracker

from ...logger import logger

__all__ = ["ActiveModuleTracker", "BaseCounter", "is_binary_tensor", "DispatchCounterMode", "FunctionCounterMode", "call_model"]

_ARROW = chr(0x2937)
_OPTIMIZER_HINTS = ("add_.", "sub_.", "mul_.", "div_.", "addcmul", "addcdiv", "lerp_", "copy_")


def _tensor_bits(x: Any) -> int:
    return int(x.numel() * x.element_size() * 8) if torch.is_tensor(x) else 0


def _collect_tensors(tree: Any) -> List[torch.Tensor]:
    return [x for x in tree_flatten(tree)[0] if torch.is_tensor(x)]


def call_model(model: nn.Module, inputs: Any) -> Any:
    """``model(*inputs)`` for tuples / lists, ``model(**inputs)`` for dicts, ``model(inputs)`` otherwise."""
    if isinstance(inputs, (tuple, list)):
        return model(*inputs)
    if isinstance(inputs, dict):
        return model(**inputs)
    return model(inputs)


def _infer_stage(func, args, kwargs, out) -> str:
    name = resolve_name(func)
    if "backward" in name:
        return "backward"
    if torch.is_grad_enabled():
        return "forward"
    if any(t.requires_grad for t in _collect_tensors((args, kwargs, out))) and any(h in name for h in _OPTIMIZER_HINTS):
        return "optimizer"
    return "forward"


def is_binary_tensor(x: torch.Tensor) -> bool:
    """True for bool tensors and tensors whose every element is 0 or 1 (costs one reduction + sync)."""
    return True if x.dtype == torch.bool else bool((x.eq(0) | x.eq(1)).all().item())


class ActiveModuleTracker(ModuleTracker):
    """``ModuleTracker`` that also keeps the *module objects* currently executing (forward or backward)."""

    def __init__(self):
        super().__init__()
        self.active_modules: Set[nn.Module] = set()

    def _get_append_fn(self, mod, name, is_bw):
        def fn(*args) -> None:
            if is_bw:
                self._maybe_set_engine_callback()
            if name in self.parents:
                logger.info("The module hierarchy tracking seems to be broken as this Module was already entered. %s during %s",
                            name, "backward" if is_bw else "forward")
            self.parents.add(name)
            self.active_modules.add(mod)
        return fn

    def _get_pop_fn(self, mod, name, is_bw):
        def fn(*args) -> None:
            if name in self.parents:
                self.parents.remove(name)
            else:
                logger.info("The Module hierarchy tracking is confused as we're exiting a Module that was never entered. %s during %s",
                            name, "backward" if is_bw else "forward")
            self.active_modules.discard(mod)
        return fn

    def _fw_pre_hook(self, mod, input) -> None:
        name = self._get_mod_name(mod)
        self._get_append_fn(mod, name, False)()
        tensors = [a for a in tree_flatten(input)[0] if isinstance(a, torch.Tensor) and a.requires_grad]
        if tensors:
            self._hooks.append(register_multi_grad_hook(tensors, self._get_pop_fn(mod, name, True)))

    def _fw_post_hook(self, mod, input, output) -> None:
        name = self._get_mod_name(mod)
        self._get_pop_fn(mod, name, False)()
        tensors = [a for a in tree_flatten(output)[0] if isinstance(a, torch.Tensor) and a.requires_grad]
        if tensors:
            self._hooks.append(register_multi_grad_hook(tensors, self._get_append_fn(mod, name, True)))


class BaseCounter:
    """``rules``: operator -> rule; ``records[scope][operator]`` accumulates; ``ignore_modules``:
    module *types* whose insides are not counted."""

    def __init__(self, extra_rules: Optional[Dict[Any, Callable]] = None, extra_ignore_modules: Optional[list] = None):
        self.records: Dict[str, Dict[Any, int]] = defaultdict(lambda: defaultdict(int))
        self.rules: Dict[Any, Callable] = dict(self.default_rules())
        self.rules.update(extra_rules or {})
        self.ignore_modules: list = list(extra_ignore_modules or [])

    def default_rules(self) -> Dict[Any, Callable]:
        return {}

    def has_rule(self, func) -> bool:
        return func in self.rules

    def count(self, func, args: tuple, kwargs: dict, out, active_modules=None, parent_names=None) -> int:
        return int(self.rules[func](args, kwargs, out))

    def record(self, scope, func, value):
        self.records[scope][func] += value

    def get_counts(self) -> Dict[str, Dict[Any, int]]:
        return {k: dict(v) for k, v in self.records.items()}

    def get_total(self) -> int:
        return sum(self.records["Global"].values())

    def reset(self):
        self.records = defaultdict(lambda: defaultdict(int))


class _CounterModeMixin:
    _label = "CounterMode"

    def _init_counters(self, counters, strict):
        self.counters = list(counters)
        self.strict = strict
        self.module_tracker = ActiveModuleTracker()

    def _skip(self, counter, func) -> bool:
        if counter.ignore_modules and any(isinstance(m, tuple(counter.ignore_modules)) for m in self.module_tracker.active_modules):
            return True
        if not counter.has_rule(func):
            if self.strict:
                raise NotImplementedError(f"{self._label}: {self.module_tracker.parents} - {resolve_name(func)} not defined by "
                                          f"{type(counter).__name__}. To disable this error, set strict=False when initializing "
                                          f"{type(counter).__name__}.")
            return True
        return False

    def _book(self, func, args, kwargs, out):
        parents = set(self.module_tracker.parents)
        active = set(self.module_tracker.active_modules)
        if logger.isEnabledFor(logging.DEBUG):
            logger.debug("%s: %s - %s", self._label, parents, resolve_name(func))
        for c in self.counters:
            if self._skip(c, func):
                continue
            value = c.count(func, args, kwargs, out, active_modules=active, parent_names=parents)
            for p in parents:
                c.record(p, func, value)
            if hasattr(c, "finalize_record"):
                c.finalize_record()


class DispatchCounterMode(_CounterModeMixin, TorchDispatchMode):
    """Counts at the ATen level (sees backward and optimizer kernels)."""
    _label = "DispatchCounterMode"

    def __init__(self, counters: List[BaseCounter], strict: bool = False):
        TorchDispatchMode.__init__(self)
        self._init_counters(counters, strict)

    def __enter__(self):
        self.module_tracker.__enter__()
        return super().__enter__()

    def __exit__(self, *args):
        ret = super().__exit__(*args)
        self.module_tracker.__exit__(*args)
        return ret

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = {} if kwargs is None else kwargs
        out = func(*args, **kwargs)
        self._book(func, args, kwargs, out)
        return out


class FunctionCounterMode(_CounterModeMixin, TorchFunctionMode):
    """Counts at the ``torch.*`` function level (rules keyed by Python callables)."""
    _label = "FunctionCounterMode"

    def __init__(self, counters: List[BaseCounter], strict: bool = False):
        TorchFunctionMode.__init__(self)
        self._init_counters(counters, strict)

    def __enter__(self):
        self.module_tracker.__enter__()
        return super().__enter__()

    def __exit__(self, *args):
        ret = super().__exit__(*args)
        self.module_tracker.__exit__(*args)
        return ret

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = {} if kwargs is None else kwargs
        out = func(*args, **kwargs)
        self._book(func, args, kwargs, out)
        return out
