"""Single-step LIF neuron (``cuda_kernel/neuron_kernel/single_step/lif.py`` of the reference).  ``decay = 1 / tau``."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .... import functional, surrogate
from . import _atgf
from .base import NeuronBPKernel, NeuronFPKernel

__all__ = ["LIFNodeFPKernel", "LIFNodeBPKernel", "cupy_single_step_lif_forward", "lif_step"]


class LIFNodeFPKernel(NeuronFPKernel):
    def __init__(self, decay_input: bool, hard_reset: bool, dtype: str):
        super().__init__(hard_reset, dtype)
        self.decay_input = decay_input
        self.kernel_name += "_decayInput" if decay_input else "_plainInput"
        self.add_param(ctype=f"const {dtype} &", cname="decay")

    def neuronal_charge(self) -> str:
        rest = "v_reset" if self.hard_reset else "0.0f"
        if self.decay_input:
            return f"h[index] = v[index] + (x[index] - (v[index] - {rest})) * decay;"
        return f"h[index] = v[index] - (v[index] - {rest}) * decay + x[index];"


class LIFNodeBPKernel(NeuronBPKernel):
    def __init__(self, decay_input: bool, surrogate_function, hard_reset: bool, detach_reset: bool, dtype: str):
        super().__init__(surrogate_function, hard_reset, detach_reset, dtype)
        self.decay_input = decay_input
        self.kernel_name += "_decayInput" if decay_input else "_plainInput"
        self.add_param(ctype=f"const {dtype} &", cname="decay")

    def grad_h_to_v(self) -> str:
        return "const float grad_h_to_v = 1.0f - decay;"

    def grad_h_to_x(self) -> str:
        return "const float grad_h_to_x = decay;" if self.decay_input else "const float grad_h_to_x = 1.0f;"


def lif_step(x: torch.Tensor, v: torch.Tensor, v_th: float, v_reset: Optional[float], decay: float, decay_input: bool,
             surrogate_function: surrogate.SurrogateFunctionBase, detach_reset: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(spike, v_next)`` through the native scan kernel with T = 1."""
    return functional.neuron.lif_step_cuda(x, v, 1.0 / decay, decay_input, v_th, v_reset, surrogate_function, detach_reset)


def cupy_single_step_lif_forward(x, v, v_th: float, v_reset: float, soft_reset: bool, decay: float, decay_input: bool, surrogate_function,
                                 detach_reset: bool = False):
    fwd = LIFNodeFPKernel(decay_input, hard_reset=not soft_reset, dtype="float")
    bwd = LIFNodeBPKernel(decay_input, surrogate_function, hard_reset=not soft_reset, detach_reset=detach_reset, dtype="float")
    s, v_next = _atgf.run(x, v, v_th, None if soft_reset else v_reset, fwd, bwd, {"decay": float(decay)})
    return s, v_next, None
