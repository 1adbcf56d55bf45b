"""Batch-norm variants for spiking networks.

* ``BatchNorm1d/2d/3d`` — step-mode wrappers; multi-step statistics are taken over
  ``T*N`` jointly.  While a gradient-checkpointed segment runs its throw-away first
  forward, running statistics are not updated (they would be counted twice).
* ``NeuNorm`` — auxiliary-neuron normalisation (stateful).
* ``ThresholdDependentBatchNorm*`` (tdBN) — ``weight`` initialised to ``alpha * v_th``.
* ``TemporalEffectiveBatchNorm*`` (TEBN) — a learnable scale per time step.
* ``BatchNormThroughTime*`` (BNTT) — a separate BN per time step.

Parity: ``spikingjelly/activation_based/layer/bn.py:29-998``.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
from torch import Tensor
from torch.nn.modules.batchnorm import _BatchNorm

from .. import base, functional

__all__ = [
    "BatchNorm1d", "BatchNorm2d", "BatchNorm3d", "NeuNorm", "ThresholdDependentBatchNorm1d",
    "ThresholdDependentBatchNorm2d", "ThresholdDependentBatchNorm3d", "TemporalEffectiveBatchNorm1d",
    "TemporalEffectiveBatchNorm2d", "TemporalEffectiveBatchNorm3d", "BatchNormThroughTime1d",
    "BatchNormThroughTime2d", "BatchNormThroughTime3d",
]


def _in_discarded_forward() -> bool:
    from ..memopt.checkpointing import in_gc_1st_forward
    return in_gc_1st_forward()


def _bn_forward(module: _BatchNorm, x: Tensor) -> Tensor:
    """``_BatchNorm.forward`` that leaves running statistics alone during the first
    (discarded) forward of a checkpointed segment."""
    if not _in_discarded_forward():
        return _BatchNorm.forward(module, x)
    saved = module.track_running_stats
    module.track_running_stats = False
    try:
        return _BatchNorm.forward(module, x)
    finally:
        module.track_running_stats = saved


def _step_bn(torch_cls, name: str, ranks, shape_txt: str):
    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, track_running_stats=True, step_mode="s",
                 **kw):
        torch_cls.__init__(self, num_features, eps, momentum, affine, track_running_stats, **kw)
        self.step_mode = step_mode

    def extra_repr(self):
        return torch_cls.extra_repr(self) + f", step_mode={self.step_mode}"

    def super_forward(self, x):
        return _bn_forward(self, x)

    def forward(self, x):
        if self.step_mode == "s":
            return _bn_forward(self, x)
        if x.dim() not in ranks:
            raise ValueError(f"expected x with shape {shape_txt}, but got x with shape {x.shape}!")
        return functional.seq_to_ann_forward(x, lambda t: _bn_forward(self, t))

    return type(name, (torch_cls, base.StepModule),
                {"__init__": __init__, "extra_repr": extra_repr, "forward": forward, "super_forward": super_forward,
                 "__module__": __name__, "__doc__": f"``torch.nn.{torch_cls.__name__}`` with ``step_mode``."})


BatchNorm1d = _step_bn(nn.BatchNorm1d, "BatchNorm1d", (3, 4), "[T, N, C, L] or [T, N, C]")
BatchNorm2d = _step_bn(nn.BatchNorm2d, "BatchNorm2d", (5,), "[T, N, C, H, W]")
BatchNorm3d = _step_bn(nn.BatchNorm3d, "BatchNorm3d", (6,), "[T, N, C, D, H, W]")


class NeuNorm(base.MemoryModule):
    """``x_t = k0 x_{t-1} + k1 sum_c s_t`` (one auxiliary neuron per pixel);
    output ``s_t - w * x_t``.  ``k1 = (1 - k0) / C^2``."""

    def __init__(self, in_channels: int, height: int, width: int, k: float = 0.9,
                 shared_across_channels: bool = False, step_mode: str = "s"):
        super().__init__()
        self.step_mode = step_mode
        self.register_memory("x", 0.0)
        self.k0 = k
        self.k1 = (1.0 - k) / in_channels ** 2
        self.w = nn.Parameter(torch.empty(1 if shared_across_channels else in_channels, height, width))
        nn.init.kaiming_uniform_(self.w, a=math.sqrt(5))

    def materialize_states(self, inputs, states, step_mode):
        if isinstance(states[0], Tensor):
            return states
        ref = inputs[0][0] if step_mode == "m" else inputs[0]
        return (torch.full_like(ref[:, :1], states[0]),)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        out, state = functional.neunorm_step(inputs[0], states[0], self.w, self.k0, self.k1)
        return (out,), (state,)

    def extra_repr(self) -> str:
        return f"shape={self.w.shape}"


class _SeqBatchNorm(_BatchNorm, base.MultiStepModule):
    """Multi-step-only BN over ``[T, N, C, *]``; ``_rank`` is the folded rank(s) accepted."""
    _ranks = ()

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._step_mode = "m"

    def _check_input_dim(self, input):
        if input.dim() not in self._ranks:
            raise ValueError(f"expect input of rank {self._ranks} after folding T into N, but get {input.shape}")

    def super_forward(self, x):
        return _bn_forward(self, x)

    def forward(self, x_seq):
        return functional.seq_to_ann_forward(x_seq, self.super_forward)


class _TdBN(_SeqBatchNorm):
    def __init__(self, alpha: float, v_th: float, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.alpha, self.v_th = alpha, v_th
        assert self.affine, "ThresholdDependentBatchNorm needs to set `affine = True`!"
        nn.init.constant_(self.weight, alpha * v_th)


class ThresholdDependentBatchNorm1d(_TdBN):
    _ranks = (2, 3)


class ThresholdDependentBatchNorm2d(_TdBN):
    _ranks = (4,)


class ThresholdDependentBatchNorm3d(_TdBN):
    _ranks = (5,)


class _TEBN(_SeqBatchNorm):
    def __init__(self, T: int, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.scale = nn.Parameter(torch.ones([T]))

    def forward(self, x_seq):
        y = super().forward(x_seq)
        return y * self.scale.view(-1, *([1] * (y.dim() - 1)))


class TemporalEffectiveBatchNorm1d(_TEBN):
    _ranks = (2, 3)


class TemporalEffectiveBatchNorm2d(_TEBN):
    _ranks = (4,)


class TemporalEffectiveBatchNorm3d(_TEBN):
    _ranks = (5,)


class _BNTT(base.MemoryModule):
    """One bias-free BN per time step; the step counter ``t`` is a memory."""
    bn_type = _BatchNorm

    def __init__(self, T: int, num_features: int, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True,
                 track_running_stats: bool = True, step_mode: str = "s"):
        super().__init__()
        self.bn_list = nn.ModuleList(
            self.bn_type(num_features, eps, momentum, affine, track_running_stats) for _ in range(T))
        for bn in self.bn_list:
            bn.bias = None
        self.T = T
        self.step_mode = step_mode
        self.register_memory("t", -1)

    def single_step_functional_forward(self, inputs, states, **kwargs):
        t = states[0] + 1
        return (_bn_forward(self.bn_list[t], inputs[0]),), (t,)


class BatchNormThroughTime1d(_BNTT):
    bn_type = nn.BatchNorm1d


class BatchNormThroughTime2d(_BNTT):
    bn_type = nn.BatchNorm2d


class BatchNormThroughTime3d(_BNTT):
    bn_type = nn.BatchNorm3d
