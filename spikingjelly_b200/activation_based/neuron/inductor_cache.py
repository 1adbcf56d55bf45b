"""Bounded, fork-safe cache of prepared multi-step graphs, keyed by neuron hyper-parameters, surrogate identity and run-time
facts (``neuron/inductor_cache.py:15-249`` of the reference, where the cached objects are ``torch.compile``-d Python time loops).

``backend="inductor"`` selects the native scan kernels in this package, so nothing has to be compiled by a tracing compiler:
``compile_graph`` keeps the callable it is given (at most 64 entries, least recently used first out, emptied in a forked
child) and returns the cached one for an equal key, which preserves the contract callers rely on: one prepared object per
configuration.  The key helpers are the reference's: a surrogate with hooks, or from outside the ``surrogate`` module, or
without both of its functional forms has no key (``None``) and is never cached."""
from __future__ import annotations

import os
import threading
from collections import OrderedDict
from typing import Any, Callable, Dict, Optional, Tuple

import torch

__all__ = ["clear", "info", "surrogate_key", "runtime_key", "surrogate_callable", "compile_graph"]

_MAX_ENTRIES = 64
_lock = threading.RLock()
_graphs: "OrderedDict[tuple, Callable]" = OrderedDict()
_stats = {"hits": 0, "misses": 0, "evictions": 0}
_pid = os.getpid()


def _forget() -> None:
    global _pid
    _graphs.clear()
    for k in _stats:
        _stats[k] = 0
    _pid = os.getpid()


if hasattr(os, "register_at_fork"):
    os.register_at_fork(after_in_child=_forget)


def _check_fork() -> None:
    if _pid != os.getpid():           # platforms without register_at_fork
        with _lock:
            _forget()


def clear() -> None:
    with _lock:
        _forget()


def info() -> Dict[str, int]:
    _check_fork()
    with _lock:
        return {"entries": len(_graphs), "max_entries": _MAX_ENTRIES, **_stats}


def surrogate_key(surrogate_function: Callable) -> Optional[Tuple[Any, ...]]:
    if any(getattr(surrogate_function, n, None) for n in ("_forward_hooks", "_forward_pre_hooks", "_backward_hooks")):
        return None
    cls = type(surrogate_function)
    own = cls.__module__.endswith("activation_based.surrogate")
    if not own or not all(any(n in k.__dict__ for k in cls.__mro__[:-1]) for n in ("spiking_function", "primitive_function")):
        return None
    params = tuple(sorted(getattr(surrogate_function, "_sg_params", {}).items()))
    return cls.__module__, cls.__qualname__, getattr(surrogate_function, "spiking", None), params


def runtime_key(*tensors: torch.Tensor) -> Tuple[Any, ...]:
    return tuple((tuple(t.shape), t.dtype, t.device, t.requires_grad) for t in tensors)


def surrogate_callable(surrogate_function: Callable) -> Callable:
    """The surrogate as a plain function of one tensor (its parameters bound), or the object itself when it has no key."""
    if surrogate_key(surrogate_function) is None:
        return surrogate_function
    cls = type(surrogate_function)
    fn = cls.spiking_function if surrogate_function.spiking else cls.primitive_function
    params = dict(surrogate_function._sg_params)
    return lambda x: fn(x, **params)


def compile_graph(cache_key: Optional[Tuple[Any, ...]], fn: Callable) -> Callable:
    _check_fork()
    if cache_key is None:
        return fn
    with _lock:
        hit = _graphs.get(cache_key)
        if hit is not None:
            _graphs.move_to_end(cache_key)
            _stats["hits"] += 1
            return hit
        _stats["misses"] += 1
        _graphs[cache_key] = fn
        while len(_graphs) > _MAX_ENTRIES:
            _graphs.popitem(last=False)
            _stats["evictions"] += 1
        return fn
