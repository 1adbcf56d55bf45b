"""Which parts of a model carry state and which can be sharded by tensor parallelism.

Result type and entry point as in ``spikingjelly/activation_based/distributed/analysis.py:15-160``; the scan itself is a
single pass that classifies every sub-module with :func:`classify`."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch.nn as nn

from ..activation_based import base
from . import _schema

__all__ = ["SNNDistributedAnalysis", "analyze_snn_distributed_capability", "linear_like_types", "classify"]

_CONVOLUTIONS = (nn.Conv1d, nn.Conv2d, nn.Conv3d)


def linear_like_types() -> tuple:
    """Module types the automatic tensor-parallel plan may shard: ``nn.Linear`` (the step-mode ``layer.Linear`` derives
    from it) and the temporal-difference linear operator of the conversion toolbox when that imports."""
    try:
        from ..activation_based.ann2snn.operators import TDLinear
    except Exception:
        return (nn.Linear,)
    return (nn.Linear, TDLinear)


def classify(module: nn.Module, linear_like: tuple) -> Optional[str]:
    """``"candidate"`` (linear-like: sharded automatically), ``"convolution"`` (only by opt-in channel sharding) or None."""
    if isinstance(module, linear_like):
        return "candidate"
    if isinstance(module, _CONVOLUTIONS):
        return "convolution"
    return None


@dataclass
class SNNDistributedAnalysis:
    memory_module_names: Tuple[str, ...]
    tensor_parallel_candidate_names: Tuple[str, ...]
    unsupported_tensor_parallel_names: Tuple[str, ...]
    notes: Tuple[str, ...]
    tensor_parallel_roots: Optional[Tuple[str, ...]] = None


def _iter_named_modules_under_roots(module: nn.Module, roots: Optional[Sequence[str]] = None) -> Iterator[Tuple[str, nn.Module]]:
    """``(path, sub-module)`` for everything below the given roots (each path once), or below the model when no roots are given."""
    everything: Dict[str, nn.Module] = dict(module.named_modules())
    if not roots:
        yield from ((path, m) for path, m in everything.items() if path)
        return
    emitted = set()
    for root in _schema.module_paths(roots, everything, "tensor_parallel_roots"):
        prefix = root + "."
        for path, m in everything.items():
            if (path == root or path.startswith(prefix)) and path not in emitted:
                emitted.add(path)
                yield path, m


def analyze_snn_distributed_capability(module: nn.Module, tensor_parallel_roots: Optional[Sequence[str]] = None) -> SNNDistributedAnalysis:
    linear_like = linear_like_types()
    stateful = tuple(path for path, m in module.named_modules() if path and isinstance(m, base.MemoryModule))
    found: Dict[str, List[str]] = {"candidate": [], "convolution": []}
    for path, m in _iter_named_modules_under_roots(module, tensor_parallel_roots):
        kind = classify(m, linear_like)
        if kind is not None:
            found[kind].append(path)
    remarks = []
    if stateful:
        remarks.append(f"{len(stateful)} stateful module(s) stay on every rank; their state takes the sharding of their input")
    if found["convolution"]:
        remarks.append(f"{len(found['convolution'])} convolution(s) are left whole by the automatic plan (channel sharding is opt-in)")
    if not found["candidate"]:
        remarks.append("nothing linear-like under the selected roots: no automatic tensor-parallel plan is possible")
    return SNNDistributedAnalysis(stateful, tuple(found["candidate"]), tuple(found["convolution"]), tuple(remarks),
                                  None if tensor_parallel_roots is None else tuple(tensor_parallel_roots))


def __getattr__(name: str):
    # ``LinearLike``: the tuple of shardable linear types, resolved on first use (the conversion toolbox imports this
    # package, so the tuple cannot be built while this module is being imported)
    if name == "LinearLike":
        return linear_like_types()
    raise AttributeError(name)
