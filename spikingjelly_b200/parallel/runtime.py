"""``SNNDistributedRuntime``: what ``apply()`` hands back — the configured model with its mesh, analysis and plan, and the
few things a training loop needs from them (``spikingjelly/activation_based/distributed/runtime.py:22-160``)."""
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

_BATCH_SHARDING_MODES = ("dp", "fsdp2", "fsdp2_tp")


@dataclass
class SNNDistributedRuntime:
    model: nn.Module
    mesh: Optional[object]
    analysis: Optional[SNNDistributedAnalysis]
    plan: SNNDistributedPlan

    # ------------------------------------------------------------------ optimizer and state
    def build_optimizer(self, optimizer_cls=torch.optim.Adam, lr: float = 1e-3, weight_decay: float = 0.0, **kwargs):
        """The plan's optimizer strategy (ZeRO-1 or plain) applied to ``optimizer_cls``."""
        return build_snn_optimizer(self.model, self.plan.mode, lr, weight_decay, self.plan.optimizer_strategy,
                                   optimizer_cls=optimizer_cls, **kwargs)

    def reset_state(self) -> None:
        """Put every stateful module back to its initial state; once per batch, after the optimizer step."""
        functional.reset_net(self.model)

    # ------------------------------------------------------------------ outputs
    @staticmethod
    def reduce_classification_output(outputs: torch.Tensor, labels: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Rate over time and class indices, leaving a sharded output sharded."""
        prepared = prepare_classification_output(outputs, labels, require_full_logits=False)
        return prepared.logits, prepared.target

    def prepare_classification_output(self, outputs, labels: torch.Tensor, *, return_metadata: bool = False):
        """Rate over time, class indices and full (gathered) logits; ``return_metadata`` returns the named tuple that also
        says whether a gather took place."""
        prepared: PreparedModelOutput = prepare_classification_output(outputs, labels, require_full_logits=True)
        return prepared if return_metadata else (prepared.logits, prepared.target)

    def forward_loss(self, criterion, images: torch.Tensor, labels: torch.Tensor):
        """``(logits, labels, criterion(logits, labels))`` with the images moved to the model's device and dtype."""
        first = next(self.model.parameters(), None)
        if first is not None:
            images = images.to(device=first.device, dtype=first.dtype)
        logits, labels = self.prepare_classification_output(self.model(images), labels)
        return logits, labels, criterion(logits, labels)

    # ------------------------------------------------------------------ data
    def prepare_dataloader(self, *, dataset, batch_size: int, shuffle: bool, num_workers: int, drop_last: bool,
                           pin_memory: bool = True) -> DataLoader:
        """A loader whose sampler splits the data over the REPLICAS of the model only: ranks that share a replica through
        tensor parallelism must be fed identical samples."""
        sampler = None
        replicas, index = 1, 0
        if dist.is_initialized():
            replicas, index = resolve_data_parallel_partition(self.mesh, self.plan.dp_mesh_dim, self.plan.mode in _BATCH_SHARDING_MODES)
        if replicas > 1:
            sampler = DistributedSampler(dataset, num_replicas=replicas, rank=index, shuffle=shuffle)
        loader = DataLoader(dataset, batch_size=batch_size, sampler=sampler, shuffle=shuffle and sampler is None,
                            num_workers=num_workers, pin_memory=pin_memory, drop_last=drop_last)
        logger.info("data loader: %s, batch %d, replica %d of %d, %d worker(s)", type(dataset).__name__, batch_size, index, replicas,
                    num_workers)
        return loader
