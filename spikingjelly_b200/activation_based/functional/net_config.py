"""Whole-network switches: reset, step mode, backend, detach.

Parity: ``spikingjelly/activation_based/functional/net_config.py`` —
``reset_net`` :98-156 (with its weak-reference module cache :22-95),
``set_step_mode`` :159-248, ``set_backend`` :251-331, ``detach_net`` :334-385.
"""
from __future__ import annotations

import weakref
from typing import Optional, Tuple, Union

import torch.nn as nn

from ...logger import logger
from .. import base

__all__ = ["collect_reset_modules", "detach_net", "invalidate_reset_cache", "reset_collected_modules",
           "reset_net", "set_backend", "set_step_mode"]

# net -> weak references of its resettable modules.  Walking ``net.modules()`` on
# every training step is measurable on deep models; the cache makes reset O(#neurons).
_cache: "weakref.WeakKeyDictionary[nn.Module, Tuple[weakref.ReferenceType, ...]]" = weakref.WeakKeyDictionary()


def _cacheable(net: nn.Module) -> bool:
    t = type(net)
    return t.__eq__ is object.__eq__ and t.__hash__ is object.__hash__


def collect_reset_modules(net: nn.Module) -> Tuple[nn.Module, ...]:
    return tuple(m for m in net.modules() if callable(getattr(m, "reset", None)))


def reset_collected_modules(modules: Tuple[nn.Module, ...]) -> None:
    for m in modules:
        if not isinstance(m, base.MemoryModule):
            logger.warning("Trying to call `reset()` of %s, which is not a MemoryModule", m)
        m.reset()


def invalidate_reset_cache(net: nn.Module) -> None:
    """Forget the cached module list of ``net`` (call after adding/removing modules)."""
    if _cacheable(net):
        _cache.pop(net, None)


def reset_net(net: nn.Module) -> None:
    """Call ``reset()`` on every module below ``net`` that has one."""
    if _cacheable(net):
        refs = _cache.get(net)
        if refs is not None:
            mods = tuple(r() for r in refs)
            if all(m is not None for m in mods):
                reset_collected_modules(mods)
                return
            _cache.pop(net, None)
    mods = collect_reset_modules(net)
    if _cacheable(net):
        _cache[net] = tuple(weakref.ref(m) for m in mods)
    reset_collected_modules(mods)


def set_step_mode(net: nn.Module, step_mode: str) -> None:
    """Set ``step_mode`` on every module that has one.  Containers that fix the step
    mode of their children (``StepModeContainer`` and the recurrent containers) are
    set themselves but not descended into."""
    from ..layer import ElementWiseRecurrentContainer, LinearRecurrentContainer, StepModeContainer
    opaque = (StepModeContainer, ElementWiseRecurrentContainer, LinearRecurrentContainer)
    stack = [net]
    while stack:
        m = stack.pop()
        if hasattr(m, "step_mode"):
            if not isinstance(m, base.StepModule):
                logger.warning("Trying to set the step mode for %s, which is not a StepModule", m)
            m.step_mode = step_mode
        if not isinstance(m, opaque):
            stack.extend(reversed(tuple(m.children())))


def set_backend(net: nn.Module, backend: str, instance: Optional[Union[type, Tuple[type, ...]]] = None) -> None:
    """Set ``backend`` on every module (of type ``instance``) that supports it; others
    keep theirs and a warning is logged."""
    instance = (nn.Module,) if instance is None else instance
    for m in net.modules():
        if not isinstance(m, instance) or not hasattr(m, "backend"):
            continue
        if not isinstance(m, base.MemoryModule):
            logger.warning("Trying to set the backend for %s, which is not a MemoryModule", m)
        supported = m.supported_backends
        if backend in supported or base.canonical_backend(backend) in supported:
            m.backend = backend
        else:
            logger.warning("%s does not support backend=%s; it will continue using backend=%s", m, backend, m.backend)


def detach_net(net: nn.Module) -> None:
    for m in net.modules():
        if hasattr(m, "detach") and callable(m.detach):
            if not isinstance(m, base.MemoryModule):
                logger.warning("Trying to call `detach()` of %s, which is not a MemoryModule", m)
            m.detach()
