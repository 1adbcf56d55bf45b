"""The logical rank grid of a job: named axes (``dp``, ``tp``, ...) whose sizes multiply to the world size.

Same role and public surface as ``spikingjelly/activation_based/distributed/topology.py:20-87`` (``world_size``, ``dims``,
``ordered_dim_names``, ``mesh_shape``, ``from_mapping``), plus :meth:`SNNDistributedTopology.axis` /
:meth:`SNNDistributedTopology.has` used by the planner."""
from __future__ import annotations

from dataclasses import dataclass
from math import prod
from types import MappingProxyType
from typing import Mapping, Optional, Tuple

from . import _schema

__all__ = ["SNNDistributedTopology"]

#: axes with a conventional position in the device mesh; any other axis follows in the order it was given
CANONICAL_AXES = ("dp", "tp", "pp", "vpp")


@dataclass(frozen=True)
class SNNDistributedTopology:
    world_size: int
    dims: Mapping[str, int]

    def __post_init__(self):
        world = _schema.positive(self.world_size, "world_size")
        if len(self.dims) == 0:
            raise ValueError("dims: a topology needs at least one axis, e.g. {'dp': 8}")
        sizes = {}
        for axis, size in self.dims.items():
            if not isinstance(axis, str) or not axis:
                raise (TypeError if not isinstance(axis, str) else ValueError)(f"dims: axis names are non-empty strings, got {axis!r}")
            if isinstance(size, float):
                raise TypeError(f"dims[{axis!r}]: expected an integer, got float")
            sizes[axis] = _schema.positive(size, f"dims[{axis!r}]")
        volume = prod(sizes.values())
        if volume != world:
            raise ValueError(f"dims: the axes {sizes} multiply to {volume}, which is not world_size = {world}")
        object.__setattr__(self, "world_size", world)
        object.__setattr__(self, "dims", MappingProxyType(sizes))

    # ------------------------------------------------------------------ queries
    def has(self, *axes: str) -> bool:
        return all(a in self.dims for a in axes)

    def axis(self, name: str) -> Optional[int]:
        """Position of ``name`` in the mesh, or ``None`` when the topology has no such axis."""
        order = self.ordered_dim_names
        return order.index(name) if name in order else None

    @property
    def ordered_dim_names(self) -> Tuple[str, ...]:
        head = tuple(a for a in CANONICAL_AXES if a in self.dims)
        return head + tuple(a for a in self.dims if a not in CANONICAL_AXES)

    @property
    def mesh_shape(self) -> Tuple[int, ...]:
        return tuple(self.dims[a] for a in self.ordered_dim_names)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_mapping(cls, dims: Mapping[str, int], *, world_size: Optional[int] = None) -> "SNNDistributedTopology":
        """Build from ``{"dp": 4, "tp": 2}``; integral floats are accepted here, ``world_size`` defaults to the product."""
        sizes = {axis: _schema.whole_number(size, f"dims[{axis!r}]") for axis, size in dims.items()}
        world = prod(sizes.values()) if world_size is None else _schema.whole_number(world_size, "world_size")
        return cls(world_size=world, dims=sizes)
