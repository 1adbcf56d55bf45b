"""Temporal augmentation for frame sequences (``spikingjelly/datasets/transform.py:9-194``)."""
from typing import Union

import numpy as np
import torch

__all__ = ["random_temporal_delete", "RandomTemporalDelete"]


def random_temporal_delete(x_seq: Union[torch.Tensor, np.ndarray], T_remain: int, batch_first: bool):
    """Keeps ``T_remain`` randomly chosen time steps, in their original order."""
    axis = 1 if batch_first else 0
    keep = np.sort(np.random.choice(x_seq.shape[axis], T_remain, replace=False))
    return x_seq[:, keep] if batch_first else x_seq[keep]


class RandomTemporalDelete(torch.nn.Module):
    def __init__(self, T_remain: int, batch_first: bool):
        super().__init__()
        self.T_remain, self.batch_first = T_remain, batch_first

    def forward(self, x_seq):
        return random_temporal_delete(x_seq, self.T_remain, self.batch_first)
