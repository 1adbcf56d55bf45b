"""Online (per-time-step) training loops: FPTT and OTTT.

Parity: ``functional/online_learning.py:18-390``.
"""
import copy
from typing import Callable, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import base
from .net_config import detach_net

__all__ = ["fptt_online_training_init_w_ra", "fptt_online_training", "ottt_online_training"]


def _params(optimizer):
    return [p for g in optimizer.param_groups for p in g["params"]]


def fptt_online_training_init_w_ra(optimizer: torch.optim.Optimizer) -> list:
    """Initial running average of the weights for FPTT (a detached copy of each)."""
    return [p.detach().clone() for p in _params(optimizer)]


def fptt_online_training(model: nn.Module, optimizer, x_seq, target_seq, f_loss_t: Callable, alpha: float,
                         w_ra: list) -> None:
    """Forward-propagation-through-time: one optimizer step per time step on the loss
    plus the dynamic regulariser ``alpha/2 * ||w - w_ra - g_prev/(2 alpha)||^2``; then the
    step is replayed (with the state restored afterwards) to refresh ``g_prev``/``w_ra``."""
    params = _params(optimizer)
    g_prev = [0.0] * len(params)
    mem_modules = tuple(m for m in model.modules() if isinstance(m, base.MemoryModule))
    T = x_seq.shape[0]
    for t in range(T):
        x_t, tgt = x_seq[t], target_seq[t]
        optimizer.zero_grad()
        loss = f_loss_t(model(x_t), tgt)
        loss = loss + (alpha / 2.0) * sum(
            F.mse_loss(p, w_ra[i] + g_prev[i] / (2.0 * alpha)) for i, p in enumerate(params))
        loss.backward()
        optimizer.step()
        detach_net(model)
        snapshot = [copy.deepcopy(m._memories) for m in mem_modules]
        optimizer.zero_grad()
        if t < T - 1:
            f_loss_t(model(x_t), tgt).backward()
            with torch.no_grad():
                for i, p in enumerate(params):
                    g_prev[i] = p.grad
                    w_ra[i] = (w_ra[i] + p) / 2.0 - p.grad / (2.0 * alpha)
        optimizer.zero_grad()
        for m, s in zip(mem_modules, snapshot):
            m._memories = s


def ottt_online_training(model: nn.Module, optimizer, x_seq, target_seq, f_loss_t: Callable,
                         online: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """Online training through time.  ``x_seq``/``target_seq`` are batch-first ``[N, T, *]``.
    ``online=True`` steps the optimizer after every time step (OTTT-O), otherwise gradients
    accumulate over the sequence (OTTT-A).  Returns (summed loss, outputs ``[N, T, *]``)."""
    x_seq, target_seq = x_seq.transpose(0, 1), target_seq.transpose(0, 1)
    total, ys = 0.0, []
    if not online:
        optimizer.zero_grad()
    for t in range(x_seq.shape[0]):
        if online:
            optimizer.zero_grad()
        y = model(x_seq[t])
        loss = f_loss_t(y, target_seq[t].contiguous())
        loss.backward()
        if online:
            optimizer.step()
        total = total + loss.detach()
        ys.append(y.detach())
    if not online:
        optimizer.step()
    return total, torch.stack(ys, dim=1)
