"""``NeuronFactory``: the recipe-side description of the spiking neuron that takes an activation's place
(``spikingjelly/activation_based/ann2snn/factories.py:9-140``)."""
from __future__ import annotations

import math
from typing import Optional, Type

import torch.nn as nn

from .. import neuron

__all__ = ["NeuronFactory"]


def _finite_real(value, what: str, *, allow_none: bool = False):
    if value is None and allow_none:
        return None
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise TypeError(f"{what}: a real number is required{' (or None)' if allow_none else ''}, got {value!r}")
    if not math.isfinite(value):
        raise ValueError(f"{what}: must be finite, got {value!r}")
    return value


class NeuronFactory:
    """Builds ``neuron_type(v_threshold=..., v_reset=..., **kwargs)`` on demand.  The default — an IF neuron with threshold 1
    and soft reset — is what rate coding wants: the activation's scale lives in the scalers placed around the neuron, and
    the soft reset keeps the charge above threshold."""

    #: set through the factory's own parameters, so they may not appear among the extra keyword arguments
    RESERVED = frozenset({"v_threshold", "v_reset"})

    def __init__(self, neuron_type: Type[nn.Module] = neuron.IFNode, v_threshold: float = 1.0, v_reset: Optional[float] = None, **kwargs):
        if not (isinstance(neuron_type, type) and issubclass(neuron_type, nn.Module)):
            raise TypeError(f"neuron_type: a subclass of nn.Module is required, got {neuron_type!r}")
        if _finite_real(v_threshold, "v_threshold") <= 0:
            raise ValueError(f"v_threshold: must be positive, got {v_threshold!r}")
        _finite_real(v_reset, "v_reset", allow_none=True)
        clash = sorted(self.RESERVED.intersection(kwargs))
        if clash:
            raise TypeError(f"{', '.join(clash)}: pass these as NeuronFactory arguments, not among the neuron's extra keyword arguments")
        self.neuron_type = neuron_type
        self.v_threshold = v_threshold
        self.v_reset = v_reset
        self.neuron_kwargs = kwargs

    @classmethod
    def neuron_kwargs_reserved_keys(cls):
        return set(cls.RESERVED)

    def create(self, scale: float) -> nn.Module:
        """A fresh neuron.  ``scale`` (the calibrated activation scale at this site) is offered to subclasses that want a
        scale-dependent threshold; the default ignores it."""
        return self.neuron_type(v_threshold=self.v_threshold, v_reset=self.v_reset, **self.neuron_kwargs)
