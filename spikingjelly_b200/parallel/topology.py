"""Logical rank grid: named dimensions whose sizes multiply to the world size.
Parity: ``spikingjelly/activation_based/distributed/topology.py:20-87``."""
from __future__ import annotations

from dataclasses import dataclass
from math import prod
from numbers import Integral
from types import MappingProxyType
from typing import Mapping, Optional, Tuple

__all__ = ["SNNDistributedTopology"]


def _as_integer(value, name: str) -> int:
    if isinstance(value, bool):
        raise TypeError(f"{name} must be an integer, but got bool.")
    if isinstance(value, Integral):
        return int(value)
    if isinstance(value, float) and value.is_integer():
        return int(value)
    raise TypeError(f"{name} must be an integer, but got {type(value).__name__}.")


@dataclass(frozen=True)
class SNNDistributedTopology:
    world_size: int
    dims: Mapping[str, int]

    def __post_init__(self):
        dims = MappingProxyType(dict(self.dims))
        object.__setattr__(self, "dims", dims)
        if not isinstance(self.world_size, Integral) or isinstance(self.world_size, bool):
            raise TypeError(f"world_size must be an integer, but got {type(self.world_size).__name__}.")
        if self.world_size <= 0:
            raise ValueError(f"world_size must be positive, but got {self.world_size}.")
        if not dims:
            raise ValueError("dims must not be empty.")
        for name, size in dims.items():
            if not isinstance(name, str):
                raise TypeError(f"Topology dimension names must be strings, but got {type(name).__name__}.")
            if not name:
                raise ValueError("Topology dimension names must be non-empty.")
            if not isinstance(size, Integral) or isinstance(size, bool):
                raise TypeError(f"Topology dimension '{name}' must be an integer, but got {type(size).__name__}.")
            if size <= 0:
                raise ValueError(f"Topology dimension '{name}' must be positive, but got {size}.")
        if prod(dims.values()) != self.world_size:
            raise ValueError(f"Topology dims {dict(dims)} multiply to {prod(dims.values())}, but world_size={self.world_size}.")

    @property
    def ordered_dim_names(self) -> Tuple[str, ...]:
        """dp, tp, pp, vpp first (in that order), then any other names in insertion order."""
        first = [n for n in ("dp", "tp", "pp", "vpp") if n in self.dims]
        return tuple(first + [n for n in self.dims if n not in first])

    @property
    def mesh_shape(self) -> Tuple[int, ...]:
        return tuple(int(self.dims[n]) for n in self.ordered_dim_names)

    @classmethod
    def from_mapping(cls, dims: Mapping[str, int], *, world_size: Optional[int] = None) -> "SNNDistributedTopology":
        norm = {k: _as_integer(v, f"Topology dimension '{k}'") for k, v in dims.items()}
        ws = prod(norm.values()) if world_size is None else _as_integer(world_size, "world_size")
        return cls(world_size=ws, dims=norm)
