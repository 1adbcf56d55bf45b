"""Data parallelism.

``prepare_snn_data_parallel`` keeps the reference's signature
(``spikingjelly/activation_based/distributed/data_parallel.py:14-35``) and returns a
``torch.nn.parallel.DistributedDataParallel`` (NCCL all-reduce of gradient buckets overlapped
with backward).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel

__all__ = ["prepare_snn_data_parallel", "unwrap_parallel_module"]


def prepare_snn_data_parallel(module: nn.Module, process_group=None, device_ids: Optional[Sequence[int]] = None,
                              broadcast_buffers: bool = False, find_unused_parameters: bool = False,
                              static_graph: bool = False) -> DistributedDataParallel:
    return DistributedDataParallel(module, device_ids=list(device_ids) if device_ids is not None else None,
                                   process_group=process_group, broadcast_buffers=broadcast_buffers,
                                   find_unused_parameters=find_unused_parameters, static_graph=static_graph)


def unwrap_parallel_module(module: nn.Module) -> nn.Module:
    return module.module if isinstance(module, DistributedDataParallel) else module
