"""Parametric LIF: functional entry point on the native scan kernel and the fragment-assembled kernel pair, whose backward
kernel also accumulates the gradient of the learnable ``decay = sigmoid(w)`` (``cuda_kernel/neuron_kernel/multi_step/plif.py``
of the reference, which reduces it in shared memory; here every thread adds its column's sum with one ``atomicAdd``)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .... import functional, surrogate
from . import _atgf
from .base import NeuronBPTTKernel, NeuronFPTTKernel

__all__ = ["ParametricLIFNodeFPTTKernel", "ParametricLIFNodeBPTTKernel", "cupy_multistep_plif_forward", "cupy_multistep_plif_backward", "plif_multi_step"]


class ParametricLIFNodeFPTTKernel(NeuronFPTTKernel):
    def __init__(self, decay_input: bool, hard_reset: bool, dtype: str):
        super().__init__(hard_reset, dtype)
        self.decay_input = decay_input
        self.kernel_name += "_decayInput" if decay_input else "_plainInput"
        self.add_param(ctype="const float *", cname="decay")

    def neuronal_charge(self) -> str:
        rest = "v_reset" if self.hard_reset else "0.0f"
        if self.decay_input:
            return f"h_seq[t] = v_v_seq[t] + (x_seq[t] - (v_v_seq[t] - {rest})) * decay[0];"
        return f"h_seq[t] = v_v_seq[t] - (v_v_seq[t] - {rest}) * decay[0] + x_seq[t];"


class ParametricLIFNodeBPTTKernel(NeuronBPTTKernel):
    needs_v_v_seq = True

    def __init__(self, decay_input: bool, surrogate_function, hard_reset: bool, detach_reset: bool, dtype: str):
        super().__init__(surrogate_function, hard_reset, detach_reset, dtype)
        self.decay_input = decay_input
        self.kernel_name += "_decayInput" if decay_input else "_plainInput"
        self.add_param(ctype="const float *", cname="decay")
        self.add_param(ctype="float *", cname="grad_decay")
        self.add_param(ctype="const float *", cname="v_v_seq")

    def grad_h_next_to_v(self) -> str:
        return "const float grad_h_next_to_v = 1.0f - decay[0];"

    def grad_h_to_x(self) -> str:
        return "const float grad_h_to_x = decay[0];" if self.decay_input else "const float grad_h_to_x = 1.0f;"

    def _extra_pre_core(self) -> str:
        return "          float grad_decay_sum = 0.0f;\n"

    def _extra_core(self) -> str:
        rest = "v_reset" if self.hard_reset else "0.0f"
        if self.decay_input:        # d h / d decay = x - (v - rest) = (h - v) / decay
            return "grad_decay_sum += grad_h * (h_seq[t] - v_v_seq[t]) / decay[0];"
        return f"grad_decay_sum += grad_h * ({rest} - v_v_seq[t]);"

    def _extra_post_core(self) -> str:
        return "          atomicAdd(grad_decay, grad_decay_sum);\n"


def plif_multi_step(x_seq: torch.Tensor, v_init: torch.Tensor, decay: torch.Tensor, decay_input: bool, v_threshold: float,
                    v_reset: Optional[float], detach_reset: bool, surrogate_function: surrogate.SurrogateFunctionBase) -> Tuple[torch.Tensor, torch.Tensor]:
    """``decay``: the one-element tensor ``sigmoid(w)``; its gradient flows back to ``w``."""
    s, _, v_seq = functional.neuron.plif_multi_step_cuda(x_seq, v_init, decay, decay_input, v_threshold, v_reset, surrogate_function,
                                                         detach_reset, store_v_seq=True)
    return s, v_seq


def cupy_multistep_plif_forward(x_seq, v_init, v_th: float, v_reset: float, soft_reset: bool, detach_reset: bool, decay: torch.Tensor,
                                decay_input: bool, surrogate_function):
    hard = not soft_reset
    fwd = ParametricLIFNodeFPTTKernel(decay_input, hard_reset=hard, dtype="float")
    bwd = ParametricLIFNodeBPTTKernel(decay_input, surrogate_function, hard_reset=hard, detach_reset=detach_reset, dtype="float")
    s, v_seq = _atgf.run(x_seq, v_init, v_th, None if soft_reset else v_reset, fwd, bwd, {"decay": decay.to(torch.float32).reshape(1)})
    return s, v_seq, None


def cupy_multistep_plif_backward(grad_spike_seq, grad_v_seq, h_seq, v_v_seq, v_th: float, v_reset: float, soft_reset: bool, detach_reset: bool,
                                 decay: torch.Tensor, decay_input: bool, surrogate_function):
    """``(grad_x_seq, grad_v_init, grad_decay)`` from saved ``h_seq`` and ``v_v_seq`` (``T + 1`` rows) through the backward kernel alone."""
    from .base import prepare_forward_meta
    bwd = ParametricLIFNodeBPTTKernel(decay_input, surrogate_function, hard_reset=not soft_reset, detach_reset=detach_reset, dtype="float")
    block = torch.zeros((h_seq.shape[0] + 1, *h_seq.shape[1:]), device=h_seq.device, dtype=h_seq.dtype)
    d = decay.detach().to(torch.float32).reshape(1)
    py_dict = {"grad_spike_seq": grad_spike_seq.contiguous(), "grad_v_seq": grad_v_seq.contiguous(), "h_seq": h_seq, "grad_x_seq": block[:-1],
               "grad_v_init": block[-1], "v_th": float(v_th), "decay": d, "grad_decay": torch.zeros_like(d), "v_v_seq": v_v_seq.contiguous()}
    if not soft_reset:
        py_dict["v_reset"] = float(v_reset)
    blocks, threads, py_dict = prepare_forward_meta(py_dict, ref="h_seq")
    bwd((blocks,), (threads,), py_dict)
    return py_dict["grad_x_seq"], py_dict["grad_v_init"], py_dict["grad_decay"]
