"""Bring the output of a (possibly sharded) classifier and its labels into the form a loss expects
(``spikingjelly/activation_based/distributed/metrics.py:10-46``): firing rate over time, class indices, full logits."""
from __future__ import annotations

from typing import NamedTuple

import torch

from .data_parallel import materialize_dtensor_output

__all__ = ["PreparedModelOutput", "prepare_classification_output"]


class PreparedModelOutput(NamedTuple):
    logits: torch.Tensor
    target: torch.Tensor
    materialized: bool


def _class_indices(target: torch.Tensor) -> torch.Tensor:
    """``[B]`` class indices from ``[B]``, ``[B, 1]`` (any number of trailing ones) or one-hot / soft ``[B, C]`` labels."""
    def drop_trailing_ones(t):
        while t.ndim > 1 and t.shape[-1] == 1:
            t = t.squeeze(-1)
        return t
    target = drop_trailing_ones(target)
    return drop_trailing_ones(target.argmax(dim=-1)) if target.ndim > 1 else target


def prepare_classification_output(output, target: torch.Tensor, *, require_full_logits: bool = True) -> PreparedModelOutput:
    """``output``: ``[T, B, C]`` (averaged over ``T``) or ``[B, C]``.  With ``require_full_logits`` a sharded output is
    gathered; ``materialized`` reports whether that happened."""
    logits = output.mean(dim=0) if output.ndim >= 3 else output
    labels = _class_indices(target)
    where = getattr(logits, "device", None)
    if where is not None and labels.device != where:
        labels = labels.to(where)
    gathered = False
    if require_full_logits:
        whole = materialize_dtensor_output(logits)
        gathered = whole is not logits
        logits = whole
    return PreparedModelOutput(logits, labels, gathered)
