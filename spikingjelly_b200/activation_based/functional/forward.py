"""Step-mode plumbing: run single-step modules over a sequence, or fold the time
axis into the batch for stateless modules.

Parity: ``spikingjelly/activation_based/functional/forward.py`` —
``multi_step_forward`` :34-85, ``t_last_multi_step_forward`` :88-142,
``chunk_multi_step_forward`` :145-227, ``seq_to_ann_forward`` :230-321,
``t_last_seq_to_ann_forward`` :324-402.
"""
from __future__ import annotations

from typing import Callable, Sequence, Tuple, Union

import torch
import torch.nn as nn
from torch import Tensor

__all__ = ["multi_step_forward", "t_last_multi_step_forward", "chunk_multi_step_forward",
           "seq_to_ann_forward", "t_last_seq_to_ann_forward"]

Module = Union[nn.Module, Sequence[nn.Module], Callable]


def _run(x, module: Module):
    """Apply ``module`` (or each module of a list in turn) to ``x`` (tensor or tuple)."""
    args = x if isinstance(x, tuple) else (x,)
    if isinstance(module, (list, tuple)):
        out = None
        for m in module:
            out = m(*args)
            args = (out,)
        return out
    return module(*args)


def _over_time(x_seq: Tensor, module: Module, dim: int) -> Tensor:
    return torch.stack([_run(x_seq.select(dim, t), module) for t in range(x_seq.shape[dim])], dim=dim)


def multi_step_forward(x_seq: Tensor, single_step_module: Module) -> Tensor:
    """``[T, N, *] -> [T, N, *]`` by calling the module once per step."""
    return _over_time(x_seq, single_step_module, 0)


def t_last_multi_step_forward(x_seq: Tensor, single_step_module: Module) -> Tensor:
    """Same for time-last layout ``[N, *, T]``."""
    return _over_time(x_seq, single_step_module, -1)


def chunk_multi_step_forward(split_size: int, x_seq: Tensor, multi_step_module: nn.Module) -> Tensor:
    """Feed a multi-step module ``split_size`` steps at a time (bounds activation memory)."""
    return torch.cat([multi_step_module(x) for x in torch.split(x_seq, split_size)], 0)


def seq_to_ann_forward(x_seq: Union[Tensor, Tuple[Tensor, ...]], stateless_module: Module):
    """Fold ``[T, N, *]`` to ``[T*N, *]`` (a view), run a stateless module once, unfold.
    This is what makes a spiking conv/linear one big GEMM over ``T x N``."""
    if isinstance(x_seq, tuple):
        lead = x_seq[0].shape[:2]
        if any(t.shape[:2] != lead for t in x_seq[1:]):
            raise ValueError("expected all tensors in x_seq to share the same [T, batch_size] leading dimensions, "
                             f"but got tensors with shapes {[tuple(t.shape) for t in x_seq]}!")
        y = _run(tuple(t.flatten(0, 1) for t in x_seq), stateless_module)
    else:
        lead = x_seq.shape[:2]
        y = _run(x_seq.flatten(0, 1), stateless_module)
    T, N = lead
    if isinstance(y, tuple):
        return tuple(t.unflatten(0, (T, N)) for t in y)
    return y.unflatten(0, (T, N))


def t_last_seq_to_ann_forward(x_seq: Tensor, stateless_module: Module):
    """Time-last variant: vectorise the module over the trailing time axis."""
    return torch.vmap(lambda x: _run(x, stateless_module), in_dims=-1, out_dims=-1)(x_seq)
