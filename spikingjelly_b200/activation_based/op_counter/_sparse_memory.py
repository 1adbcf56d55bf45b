"""Byte accounting for tensors that hardware would access sparsely: a tensor counts as sparse when it is boolean /
binary or when at least ``zero_ratio_threshold`` of it is zero (``op_counter/_sparse_memory.py:19-250``)."""
from __future__ import annotations

from typing import Any

import torch

from .base import is_binary_tensor

__all__ = ["active_element_count", "dense_bytes", "dense_bytes_tree", "is_sparse_access_tensor", "sparse_bytes", "sparse_bytes_tree"]


def active_element_count(x: torch.Tensor) -> int:
    return int(x.count_nonzero().item())


def dense_bytes(x: torch.Tensor) -> int:
    return int(x.numel()) * int(x.element_size())


def sparse_bytes(x: torch.Tensor) -> int:
    return active_element_count(x) * int(x.element_size())


def is_sparse_access_tensor(x: torch.Tensor, *, zero_ratio_threshold: float = 0.5) -> bool:
    if x.numel() == 0 or x.is_meta:
        return False
    if x.dtype == torch.bool or is_binary_tensor(x):
        return True
    return 1.0 - active_element_count(x) / float(x.numel()) >= zero_ratio_threshold


def _leaves(tree: Any):
    if torch.is_tensor(tree):
        yield tree
    elif isinstance(tree, (tuple, list)):
        for item in tree:
            yield from _leaves(item)
    elif isinstance(tree, dict):
        for item in tree.values():
            yield from _leaves(item)


def dense_bytes_tree(tree: Any) -> int:
    return sum(dense_bytes(t) for t in _leaves(tree))


def sparse_bytes_tree(tree: Any, *, zero_ratio_threshold: float = 0.5) -> int:
    return sum(sparse_bytes(t) if is_sparse_access_tensor(t, zero_ratio_threshold=zero_ratio_threshold) else dense_bytes(t)
               for t in _leaves(tree))
