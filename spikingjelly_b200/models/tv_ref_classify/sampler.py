"""Repeated-augmentation sampler: every rank sees ``repetitions`` differently augmented copies of a
shared subset, so that one optimisation step mixes several views of the same images.

Parity: ``spikingjelly/activation_based/model/tv_ref_classify/sampler.py:8-68``.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

__all__ = ["RASampler"]


class RASampler(torch.utils.data.Sampler):
    def __init__(self, dataset, num_replicas=None, rank=None, shuffle=True, seed=0, repetitions=3):
        if num_replicas is None or rank is None:
            if not (dist.is_available() and dist.is_initialized()):
                raise RuntimeError("Requires distributed package to be available!")
            num_replicas = dist.get_world_size() if num_replicas is None else num_replicas
            rank = dist.get_rank() if rank is None else rank
        self.dataset, self.num_replicas, self.rank = dataset, num_replicas, rank
        self.shuffle, self.seed, self.repetitions, self.epoch = shuffle, seed, repetitions, 0
        self.num_samples = int(math.ceil(len(dataset) * float(repetitions) / num_replicas))
        self.total_size = self.num_samples * num_replicas
        # each rank only consumes about 1/num_replicas of the *un-repeated* dataset per epoch, in multiples of 256
        self.num_selected_samples = int(math.floor(len(dataset) // 256 * 256 / num_replicas))

    def __iter__(self):
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self.epoch)
            order = torch.randperm(len(self.dataset), generator=g).tolist()
        else:
            order = list(range(len(self.dataset)))
        order = [i for i in order for _ in range(self.repetitions)]
        order += order[: self.total_size - len(order)]
        mine = order[self.rank: self.total_size: self.num_replicas]
        return iter(mine[: self.num_selected_samples])

    def __len__(self):
        return self.num_selected_samples

    def set_epoch(self, epoch: int):
        self.epoch = epoch
