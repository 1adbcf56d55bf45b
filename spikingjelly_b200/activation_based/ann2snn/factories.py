"""``NeuronFactory``: how a conversion recipe builds the neuron that replaces an activation.
Parity: ``spikingjelly/activation_based/ann2snn/factories.py:9-140``."""
from __future__ import annotations

import math
from typing import Optional, Type

import torch.nn as nn

from .. import neuron

__all__ = ["NeuronFactory"]


class NeuronFactory:
    """``create(scale)`` returns ``neuron_type(v_threshold=..., v_reset=..., **kwargs)``; the default is a
    soft-reset IF neuron with threshold 1 (the activation scale is applied by the scalers around it)."""

    def __init__(self, neuron_type: Type[nn.Module] = neuron.IFNode, v_threshold: float = 1.0, v_reset: Optional[float] = None, **kwargs):
        if not isinstance(neuron_type, type) or not issubclass(neuron_type, nn.Module):
            raise TypeError(f"neuron_type must be an nn.Module subclass, but got {neuron_type!r}.")
        if not isinstance(v_threshold, (int, float)) or isinstance(v_threshold, bool):
            raise TypeError(f"v_threshold must be a real number, got {type(v_threshold).__name__}.")
        if not math.isfinite(float(v_threshold)) or not v_threshold > 0:
            raise ValueError(f"v_threshold must be finite and positive, got {v_threshold}.")
        if v_reset is not None and (not isinstance(v_reset, (int, float)) or isinstance(v_reset, bool)):
            raise TypeError(f"v_reset must be None or a real number, got {v_reset!r}.")
        if v_reset is not None and not math.isfinite(float(v_reset)):
            raise ValueError(f"v_reset must be finite, got {v_reset}.")
        reserved = self.neuron_kwargs_reserved_keys() & kwargs.keys()
        if reserved:
            raise TypeError(f"neuron kwargs contain reserved key(s): {', '.join(sorted(reserved))}. Use NeuronFactory parameters instead.")
        self.neuron_type, self.v_threshold, self.v_reset, self.neuron_kwargs = neuron_type, v_threshold, v_reset, kwargs

    @staticmethod
    def neuron_kwargs_reserved_keys():
        return {"v_threshold", "v_reset"}

    def create(self, scale: float) -> nn.Module:
        return self.neuron_type(v_threshold=self.v_threshold, v_reset=self.v_reset, **self.neuron_kwargs)
