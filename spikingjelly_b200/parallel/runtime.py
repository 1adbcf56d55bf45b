"""``SNNDistributedRuntime``: what ``apply()`` returns — configured model, mesh, analysis and plan, with
helpers for the optimizer, state reset, classification outputs and data loading.
Parity: ``spikingjelly/activation_based/distributed/runtime.py:22-160``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler

from ..activation_based import functional
from ..logger import logger
from .analysis import SNNDistributedAnalysis
from .mesh import resolve_data_parallel_partition
from .metrics import PreparedModelOutput, prepare_classification_output
from .optimizer import build_snn_optimizer
from .planner import SNNDistributedPlan

__all__ = ["SNNDistributedRuntime"]


@dataclass
class SNNDistributedRuntime:
    model: nn.Module
    mesh: Optional[object]
    analysis: Optional[SNNDistributedAnalysis]
    plan: SNNDistributedPlan

    def build_optimizer(self, optimizer_cls=torch.optim.Adam, lr: float = 1e-3, weight_decay: float = 0.0, **kwargs):
        return build_snn_optimizer(self.model, mode=self.plan.mode, optimizer_cls=optimizer_cls, lr=lr, weight_decay=weight_decay,
                                   optimizer_sharding=self.plan.optimizer_strategy, **kwargs)

    def reset_state(self):
        """Reset every stateful module (call once per batch, after the optimizer step)."""
        functional.reset_net(self.model)

    @staticmethod
    def reduce_classification_output(outputs: torch.Tensor, labels: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        p = prepare_classification_output(outputs, labels, require_full_logits=False)
        return p.logits, p.target

    def prepare_classification_output(self, outputs, labels: torch.Tensor, *, return_metadata: bool = False):
        p = prepare_classification_output(outputs, labels, require_full_logits=True)
        return p if return_metadata else (p.logits, p.target)

    def forward_loss(self, criterion, images: torch.Tensor, labels: torch.Tensor):
        try:
            ref = next(self.model.parameters())
            dtype, device = ref.dtype, ref.device
        except StopIteration:
            dtype, device = torch.float32, torch.device("cpu")
        outputs, labels = self.prepare_classification_output(self.model(images.to(device=device, dtype=dtype)), labels)
        return outputs, labels, criterion(outputs, labels)

    def prepare_dataloader(self, *, dataset, batch_size: int, shuffle: bool, num_workers: int, drop_last: bool,
                           pin_memory: bool = True) -> DataLoader:
        """A ``DistributedSampler`` over the data-parallel replicas only (tensor-parallel ranks of one
        replica must see the same samples)."""
        sampler, replicas, rank = None, 1, 0
        if dist.is_initialized():
            replicas, rank = resolve_data_parallel_partition(self.mesh, dp_mesh_dim=self.plan.dp_mesh_dim,
                                                             sharded_by_data_parallel=self.plan.mode in ("dp", "fsdp2", "fsdp2_tp"))
            if replicas > 1:
                sampler = DistributedSampler(dataset, num_replicas=replicas, rank=rank, shuffle=shuffle)
        loader = DataLoader(dataset, batch_size=batch_size, sampler=sampler, shuffle=shuffle if sampler is None else False,
                            num_workers=num_workers, pin_memory=pin_memory, drop_last=drop_last)
        logger.info("distributed_dataloader_prepared dataset=%s batch_size=%s num_workers=%s sampler=%s replicas=%s rank=%s "
                    "drop_last=%s pin_memory=%s", type(dataset).__name__, batch_size, num_workers,
                    type(sampler).__name__ if sampler is not None else None, replicas, rank, drop_last, pin_memory)
        return loader
