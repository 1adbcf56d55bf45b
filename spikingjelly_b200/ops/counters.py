"""Counts launches of this package's own CUDA kernels (the Python entry points bump the
counter by the number of kernels they enqueue).  Used by benchmarks to report how much of a
step ran in native code."""
_count = 0
_by_name: dict = {}


def bump(name: str, n: int = 1) -> None:
    global _count
    _count += n
    _by_name[name] = _by_name.get(name, 0) + n


def reset() -> None:
    global _count
    _count = 0
    _by_name.clear()


def total() -> int:
    return _count


def by_name() -> dict:
    return dict(_by_name)
