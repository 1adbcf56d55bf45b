"""Small helpers (``functional/misc.py:19-364``)."""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

__all__ = ["set_threshold_margin", "redundant_one_hot", "first_spike_index",
           "kaiming_normal_conv_linear_weight", "delay"]


def set_threshold_margin(output_layer, label_one_hot: Tensor, eval_threshold=1.0, threshold0=0.9, threshold1=1.1):
    """Training: the target neuron gets a higher threshold (``threshold1``) than the others
    (``threshold0``) so that it must be driven harder; evaluation uses ``eval_threshold``."""
    if output_layer.training:
        th = torch.ones_like(label_one_hot) * threshold0
        th[label_one_hot == 1] = threshold1
        output_layer.v_threshold = th
    else:
        output_layer.v_threshold = eval_threshold


def redundant_one_hot(labels: Tensor, num_classes: int, n: int):
    """One-hot where each class owns ``n`` consecutive output neurons."""
    return F.one_hot(labels, num_classes).repeat_interleave(n, dim=-1).to(torch.get_default_dtype())


def first_spike_index(spikes: Tensor):
    """Boolean mask, true only at the first spike along the last (time) axis."""
    return (spikes != 0) & (spikes.cumsum(dim=-1) == 1)


def kaiming_normal_conv_linear_weight(net: nn.Module):
    for m in net.modules():
        if isinstance(m, (nn.Conv1d, nn.Conv2d, nn.Conv3d, nn.Linear)):
            nn.init.kaiming_normal_(m.weight, a=math.sqrt(5))


def delay(x_seq: Tensor, delay_steps: int):
    """Shift a sequence ``delay_steps`` steps into the future, zero-filling the head."""
    if delay_steps == 0:
        return x_seq
    if delay_steps >= x_seq.shape[0]:
        return torch.zeros_like(x_seq)
    return torch.cat((torch.zeros_like(x_seq[:delay_steps]), x_seq[:-delay_steps]))
