"""What in a model is stateful and what can be tensor-parallel.
Parity: ``spikingjelly/activation_based/distributed/analysis.py:15-160``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Optional, Sequence, Tuple

import torch.nn as nn

from ..activation_based import base

__all__ = ["SNNDistributedAnalysis", "analyze_snn_distributed_capability", "linear_like_types"]


def linear_like_types() -> tuple:
    """``nn.Linear`` (which includes the step-mode ``layer.Linear``) and, when the conversion toolbox
    is importable, the temporal-difference linear operator."""
    try:
        from ..activation_based.ann2snn.operators import TDLinear
        return (nn.Linear, TDLinear)
    except Exception:
        return (nn.Linear,)


@dataclass
class SNNDistributedAnalysis:
    memory_module_names: Tuple[str, ...]
    tensor_parallel_candidate_names: Tuple[str, ...]
    unsupported_tensor_parallel_names: Tuple[str, ...]
    notes: Tuple[str, ...]
    tensor_parallel_roots: Optional[Tuple[str, ...]] = None


def _iter_named_modules_under_roots(module: nn.Module, roots: Optional[Sequence[str]] = None) -> Iterable[Tuple[str, nn.Module]]:
    if not roots:
        yield from ((n, m) for n, m in module.named_modules() if n)
        return
    named = dict(module.named_modules())
    seen = set()
    for root in roots:
        if not root:
            raise ValueError("tensor_parallel_roots entries must be non-empty module paths; pass None or omit the argument "
                             "to scan the full model.")
        if root not in named:
            raise KeyError(f"tensor_parallel_roots contains unknown module path '{root}'.")
        for sub, child in named[root].named_modules():
            full = root if not sub else f"{root}.{sub}"
            if full not in seen:
                seen.add(full)
                yield full, child


def analyze_snn_distributed_capability(module: nn.Module, tensor_parallel_roots: Optional[Sequence[str]] = None) -> SNNDistributedAnalysis:
    linear_like = linear_like_types()
    memory = [n for n, m in module.named_modules() if n and isinstance(m, base.MemoryModule)]
    candidates, unsupported = [], []
    for name, child in _iter_named_modules_under_roots(module, tensor_parallel_roots):
        if isinstance(child, linear_like):
            candidates.append(name)
        elif isinstance(child, (nn.Conv1d, nn.Conv2d, nn.Conv3d)):
            unsupported.append(name)
    notes = []
    if memory:
        notes.append("Stateful neuron modules remain local/replicated; their state follows the sharding of their input.")
    if unsupported:
        notes.append("Convolutions are not sharded automatically; only Linear-like modules are auto-parallelized "
                     "(channel sharding of convolution stacks is opt-in).")
    if not candidates:
        notes.append("No Linear-like tensor-parallel candidates were found under the selected roots.")
    return SNNDistributedAnalysis(tuple(memory), tuple(candidates), tuple(unsupported), tuple(notes),
                                  tuple(tensor_parallel_roots) if tensor_parallel_roots is not None else None)
