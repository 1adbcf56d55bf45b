"""Optimizer construction for a configured model, with optional ZeRO-1 sharding of the optimizer state
(``spikingjelly/activation_based/distributed/optimizer.py:11-95``)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..logger import logger
from . import _schema

try:
    from torch.distributed.optim import ZeroRedundancyOptimizer
except ImportError:                                       # pragma: no cover
    ZeroRedundancyOptimizer = None
ZERO_REDUNDANCY_OPTIMIZER_AVAILABLE = ZeroRedundancyOptimizer is not None

__all__ = ["ZERO_REDUNDANCY_OPTIMIZER_AVAILABLE", "build_snn_optimizer"]


def _why_not_zero(mode: str) -> Optional[str]:
    if mode != "dp":
        return f"it needs every rank to hold every parameter, i.e. mode 'dp' (got {mode!r})"
    if not dist.is_initialized():
        return "there is no process group to shard over"
    if not ZERO_REDUNDANCY_OPTIMIZER_AVAILABLE:
        return "this PyTorch build has no ZeroRedundancyOptimizer"
    return None


def build_snn_optimizer(module: nn.Module, mode: str, lr: float, weight_decay: float = 0.0, optimizer_sharding: str = "none",
                        foreach: Optional[bool] = None, optimizer_cls=torch.optim.Adam, **optimizer_kwargs):
    """``optimizer_cls(module.parameters(), lr, weight_decay, ...)``; with ``optimizer_sharding="zero"`` the same optimizer
    wrapped so that each data-parallel rank keeps 1/world of its state."""
    sharding = _schema.one_of(optimizer_sharding, ("none", "zero"), "optimizer_sharding")
    settings = dict(optimizer_kwargs, lr=lr, weight_decay=weight_decay)
    if foreach is not None:
        settings["foreach"] = foreach
    if sharding == "zero":
        obstacle = _why_not_zero(mode)
        if obstacle is not None:
            raise (ValueError if mode != "dp" else RuntimeError)(f"optimizer_sharding='zero' cannot be used: {obstacle}")
        optimizer = ZeroRedundancyOptimizer(module.parameters(), optimizer_class=optimizer_cls, **settings)
    else:
        optimizer = optimizer_cls(module.parameters(), **settings)
    logger.info("optimizer: %s (mode=%s, state sharding=%s, lr=%g, weight decay=%g)", type(optimizer).__name__, mode, sharding, lr, weight_decay)
    return optimizer
