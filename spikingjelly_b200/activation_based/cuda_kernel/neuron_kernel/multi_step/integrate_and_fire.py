"""IF neuron: the functional entry point on the native scan kernel and the fragment-assembled kernel pair
(``cuda_kernel/neuron_kernel/multi_step/integrate_and_fire.py`` of the reference)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .... import functional, surrogate
from . import _atgf
from .base import NeuronBPTTKernel, NeuronFPTTKernel

__all__ = ["IFNodeFPTTKernel", "IFNodeBPTTKernel", "cupy_multistep_if_forward", "cupy_multistep_if_backward", "if_multi_step"]


class IFNodeFPTTKernel(NeuronFPTTKernel):
    def neuronal_charge(self) -> str:
        return "h_seq[t] = x_seq[t] + v_v_seq[t];"


class IFNodeBPTTKernel(NeuronBPTTKernel):
    def grad_h_next_to_v(self) -> str:
        return "const float grad_h_next_to_v = 1.0f;"

    def grad_h_to_x(self) -> str:
        return "const float grad_h_to_x = 1.0f;"


def if_multi_step(x_seq: torch.Tensor, v_init: torch.Tensor, v_threshold: float, v_reset: Optional[float], detach_reset: bool,
                  surrogate_function: surrogate.SurrogateFunctionBase) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(spike_seq, v_seq)`` on the native scan kernel (any shape ``[T, ...]``, fp32 / fp16 / bf16)."""
    s, _, v_seq = functional.neuron.if_multi_step_cuda(x_seq, v_init, v_threshold, v_reset, surrogate_function, detach_reset, store_v_seq=True)
    return s, v_seq


def cupy_multistep_if_forward(x_seq, v_init, v_th: float, v_reset: float, soft_reset: bool, detach_reset: bool, surrogate_function):
    """The fragment-assembled pair, differentiable: ``(spike_seq, v_seq, h_seq)``.  The reference's operator takes a surrogate id
    in the last position; here the surrogate object itself is passed (its derivative is emitted into the backward kernel)."""
    hard = not soft_reset
    fwd = IFNodeFPTTKernel(hard_reset=hard, dtype="float")
    bwd = IFNodeBPTTKernel(surrogate_function, hard_reset=hard, detach_reset=detach_reset, dtype="float")
    s, v_seq = _atgf.run(x_seq, v_init, v_th, None if soft_reset else v_reset, fwd, bwd)
    return s, v_seq, None


def cupy_multistep_if_backward(grad_spike_seq, grad_v_seq, h_seq, v_th: float, v_reset: float, soft_reset: bool, detach_reset: bool,
                               surrogate_function):
    """``(grad_x_seq, grad_v_init)`` from saved ``h_seq`` through the backward kernel alone."""
    from .base import prepare_forward_meta
    bwd = IFNodeBPTTKernel(surrogate_function, hard_reset=not soft_reset, detach_reset=detach_reset, dtype="float")
    block = torch.zeros((h_seq.shape[0] + 1, *h_seq.shape[1:]), device=h_seq.device, dtype=h_seq.dtype)
    py_dict = {"grad_spike_seq": grad_spike_seq.contiguous(), "grad_v_seq": grad_v_seq.contiguous(), "h_seq": h_seq, "grad_x_seq": block[:-1],
               "grad_v_init": block[-1], "v_th": float(v_th)}
    if not soft_reset:
        py_dict["v_reset"] = float(v_reset)
    blocks, threads, py_dict = prepare_forward_meta(py_dict, ref="h_seq")
    bwd((blocks,), (threads,), py_dict)
    return py_dict["grad_x_seq"], py_dict["grad_v_init"]
