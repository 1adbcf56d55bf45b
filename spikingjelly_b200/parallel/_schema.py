"""Small argument checkers shared by the distributed vocabulary (topology, configuration, planner).

Every checker returns the normalised value and raises with a message that names the offending field, so the data
classes built on them carry no validation code of their own."""
from __future__ import annotations

from numbers import Integral
from typing import Iterable, Optional, Sequence

__all__ = ["whole_number", "positive", "one_of", "axis_index", "module_paths"]


def whole_number(value, field: str) -> int:
    """An ``int`` from an integer or an integral float; booleans and everything else are type errors."""
    if isinstance(value, bool) or not isinstance(value, (Integral, float)):
        raise TypeError(f"{field}: expected an integer, got {type(value).__name__} ({value!r})")
    if isinstance(value, float):
        if not value.is_integer():
            raise TypeError(f"{field}: expected an integer, got the fractional value {value!r}")
        return int(value)
    return int(value)


def positive(value, field: str) -> int:
    n = whole_number(value, field)
    if n < 1:
        raise ValueError(f"{field}: must be at least 1, got {n}")
    return n


def one_of(value: str, allowed: Sequence[str], field: str) -> str:
    """Case-insensitive membership test; returns the lower-cased value."""
    if not isinstance(value, str):
        raise TypeError(f"{field}: expected one of {tuple(allowed)}, got {type(value).__name__}")
    low = value.lower()
    if low not in allowed:
        raise ValueError(f"{field}: {value!r} is not one of {tuple(allowed)}")
    return low


def axis_index(value: Optional[int], ndim: int, field: str, *, optional: bool = False) -> Optional[int]:
    if value is None:
        if optional:
            return None
        raise ValueError(f"{field}: a mesh axis index is required")
    i = whole_number(value, field)
    if not 0 <= i < ndim:
        raise ValueError(f"{field}: axis {i} does not exist on a mesh with {ndim} axis/axes")
    return i


def module_paths(paths: Optional[Iterable[str]], known: Iterable[str], field: str) -> Optional[tuple]:
    """Dotted module paths that must all exist in ``known``; ``None`` stays ``None``."""
    if paths is None:
        return None
    known = set(known)
    out = []
    for p in paths:
        if not isinstance(p, str) or not p:
            raise ValueError(f"{field}: entries are non-empty dotted module paths (omit the argument to cover the whole model)")
        if p not in known:
            raise KeyError(f"{field}: the model has no sub-module {p!r}")
        out.append(p)
    return tuple(out)
