"""Single-step IF neuron (``cuda_kernel/neuron_kernel/single_step/integrate_and_fire.py`` of the reference)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .... import functional, surrogate
from . import _atgf
from .base import NeuronBPKernel, NeuronFPKernel

__all__ = ["IFNodeFPKernel", "IFNodeBPKernel", "cupy_single_step_if_forward", "if_step"]


class IFNodeFPKernel(NeuronFPKernel):
    def neuronal_charge(self) -> str:
        return "h[index] = x[index] + v[index];"


class IFNodeBPKernel(NeuronBPKernel):
    def grad_h_to_v(self) -> str:
        return "const float grad_h_to_v = 1.0f;"

    def grad_h_to_x(self) -> str:
        return "const float grad_h_to_x = 1.0f;"


def if_step(x: torch.Tensor, v: torch.Tensor, v_th: float, v_reset: Optional[float], surrogate_function: surrogate.SurrogateFunctionBase,
            detach_reset: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(spike, v_next)`` through the native scan kernel with T = 1."""
    return functional.neuron.if_step_cuda(x, v, v_th, v_reset, surrogate_function, detach_reset)


def cupy_single_step_if_forward(x, v, v_th: float, v_reset: float, soft_reset: bool, surrogate_function, detach_reset: bool = False):
    """The fragment-assembled pair, differentiable: ``(spike, v_next, h)`` (``h`` stays inside the function)."""
    fwd = IFNodeFPKernel(hard_reset=not soft_reset, dtype="float")
    bwd = IFNodeBPKernel(surrogate_function, hard_reset=not soft_reset, detach_reset=detach_reset, dtype="float")
    s, v_next = _atgf.run(x, v, v_th, None if soft_reset else v_reset, fwd, bwd)
    return s, v_next, None
