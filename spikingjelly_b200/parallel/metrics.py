"""Classification outputs of a (possibly sharded) model: mean over time, label normalisation and
materialisation of sharded outputs.  Parity: ``spikingjelly/activation_based/distributed/metrics.py:10-46``."""
from __future__ import annotations

from typing import NamedTuple

import torch

from .data_parallel import materialize_dtensor_output

__all__ = ["PreparedModelOutput", "prepare_classification_output"]


class PreparedModelOutput(NamedTuple):
    logits: torch.Tensor
    target: torch.Tensor
    materialized: bool


def _labels(target: torch.Tensor) -> torch.Tensor:
    while target.ndim > 1 and target.shape[-1] == 1:
        target = target.squeeze(-1)
    if target.ndim > 1:                                   # one-hot / soft labels
        target = target.argmax(dim=-1)
        while target.ndim > 1 and target.shape[-1] == 1:
            target = target.squeeze(-1)
    return target


def prepare_classification_output(output, target: torch.Tensor, *, require_full_logits: bool = True) -> PreparedModelOutput:
    if output.ndim >= 3:
        output = output.mean(dim=0)                       # [T, B, C] -> rate
    target = _labels(target)
    dev = getattr(output, "device", None)
    if dev is not None and target.device != dev:
        target = target.to(device=dev)
    materialized = False
    if require_full_logits:
        full = materialize_dtensor_output(output)
        materialized, output = full is not output, full
    return PreparedModelOutput(output, target, materialized)
