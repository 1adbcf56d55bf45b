"""LIF neuron: functional entry point on the native scan kernel and the fragment-assembled kernel pair
(``cuda_kernel/neuron_kernel/multi_step/lif.py`` of the reference).  ``decay = 1 / tau``."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .... import functional, surrogate
from . import _atgf
from .base import NeuronBPTTKernel, NeuronFPTTKernel

__all__ = ["LIFNodeFPTTKernel", "LIFNodeBPTTKernel", "cupy_multistep_lif_forward", "cupy_multistep_lif_backward", "lif_multi_step"]


class LIFNodeFPTTKernel(NeuronFPTTKernel):
    def __init__(self, decay_input: bool, hard_reset: bool, dtype: str):
        super().__init__(hard_reset, dtype)
        self.decay_input = decay_input
        self.kernel_name += "_decayInput" if decay_input else "_plainInput"
        self.add_param(ctype=f"const {dtype} &", cname="decay")

    def neuronal_charge(self) -> str:
        rest = "v_reset" if self.hard_reset else "0.0f"
        if self.decay_input:
            return f"h_seq[t] = v_v_seq[t] + (x_seq[t] - (v_v_seq[t] - {rest})) * decay;"
        return f"h_seq[t] = v_v_seq[t] - (v_v_seq[t] - {rest}) * decay + x_seq[t];"


class LIFNodeBPTTKernel(NeuronBPTTKernel):
    def __init__(self, decay_input: bool, surrogate_function, hard_reset: bool, detach_reset: bool, dtype: str):
        super().__init__(surrogate_function, hard_reset, detach_reset, dtype)
        self.decay_input = decay_input
        self.kernel_name += "_decayInput" if decay_input else "_plainInput"
        self.add_param(ctype=f"const {dtype} &", cname="decay")

    def grad_h_next_to_v(self) -> str:
        return "const float grad_h_next_to_v = 1.0f - decay;"

    def grad_h_to_x(self) -> str:
        return "const float grad_h_to_x = decay;" if self.decay_input else "const float grad_h_to_x = 1.0f;"


def lif_multi_step(x_seq: torch.Tensor, v_init: torch.Tensor, decay_input: bool, tau: float, v_threshold: float, v_reset: Optional[float],
                   detach_reset: bool, surrogate_function: surrogate.SurrogateFunctionBase) -> Tuple[torch.Tensor, torch.Tensor]:
    s, _, v_seq = functional.neuron.lif_multi_step_cuda(x_seq, v_init, tau, decay_input, v_threshold, v_reset, surrogate_function, detach_reset,
                                                        store_v_seq=True)
    return s, v_seq


def cupy_multistep_lif_forward(x_seq, v_init, v_th: float, v_reset: float, soft_reset: bool, detach_reset: bool, decay: float,
                               decay_input: bool, surrogate_function):
    """The fragment-assembled pair, differentiable: ``(spike_seq, v_seq, h_seq)`` (``h_seq`` is kept inside the function)."""
    hard = not soft_reset
    fwd = LIFNodeFPTTKernel(decay_input, hard_reset=hard, dtype="float")
    bwd = LIFNodeBPTTKernel(decay_input, surrogate_function, hard_reset=hard, detach_reset=detach_reset, dtype="float")
    s, v_seq = _atgf.run(x_seq, v_init, v_th, None if soft_reset else v_reset, fwd, bwd, {"decay": float(decay)})
    return s, v_seq, None


def cupy_multistep_lif_backward(grad_spike_seq, grad_v_seq, h_seq, v_th: float, v_reset: float, soft_reset: bool, detach_reset: bool,
                                decay: float, decay_input: bool, surrogate_function):
    """``(grad_x_seq, grad_v_init)`` from saved ``h_seq`` through the backward kernel alone."""
    from .base import prepare_forward_meta
    bwd = LIFNodeBPTTKernel(decay_input, surrogate_function, hard_reset=not soft_reset, detach_reset=detach_reset, dtype="float")
    block = torch.zeros((h_seq.shape[0] + 1, *h_seq.shape[1:]), device=h_seq.device, dtype=h_seq.dtype)
    py_dict = {"grad_spike_seq": grad_spike_seq.contiguous(), "grad_v_seq": grad_v_seq.contiguous(), "h_seq": h_seq, "grad_x_seq": block[:-1],
               "grad_v_init": block[-1], "v_th": float(v_th), "decay": float(decay)}
    if not soft_reset:
        py_dict["v_reset"] = float(v_reset)
    blocks, threads, py_dict = prepare_forward_meta(py_dict, ref="h_seq")
    bwd((blocks,), (threads,), py_dict)
    return py_dict["grad_x_seq"], py_dict["grad_v_init"]
