"""One autograd function for every fragment-assembled kernel pair: runs the forward kernel, keeps ``h_seq`` (and what the
backward kernel's extra parameters need), runs the backward kernel."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import NeuronATGFBase, NeuronBPTTKernel, NeuronFPTTKernel


class KernelPairFunction(torch.autograd.Function):
    """``apply(x_seq [T, N], v_init [N], v_th, v_reset | None, forward_kernel, backward_kernel, extra)``; ``extra`` maps the
    kernels' additional parameter names to values (a one-element tensor parameter that needs a gradient goes first and gets
    its gradient from the backward kernel's ``grad_<name>`` buffer).  Returns ``(spike_seq, v_seq)``."""

    @staticmethod
    def forward(ctx, x_seq, v_init, v_th: float, v_reset: Optional[float], forward_kernel: NeuronFPTTKernel,
                backward_kernel: NeuronBPTTKernel, extra: Dict, *extra_tensors):
        py_dict = {"x_seq": x_seq, "v_init": v_init, "v_th": v_th, "v_reset": v_reset, **extra}
        requires_grad, blocks, threads, py_dict = NeuronATGFBase.pre_forward(py_dict)
        forward_kernel((blocks,), (threads,), py_dict)
        saved = [py_dict["h_seq"]]
        if getattr(backward_kernel, "needs_v_v_seq", False):
            saved.append(py_dict["v_v_seq"])
        NeuronATGFBase.ctx_save(ctx, requires_grad, *saved, *extra_tensors, blocks=blocks, threads=threads, numel=py_dict["numel"], N=py_dict["N"],
                                v_th=v_th, v_reset=v_reset, backward_kernel=backward_kernel, extra=extra, n_saved=len(saved))
        return py_dict["spike_seq"], py_dict["v_v_seq"][1:]

    @staticmethod
    def backward(ctx, grad_spike_seq, grad_v_seq):
        kernel, blocks, threads, py_dict = NeuronATGFBase.pre_backward(ctx, grad_spike_seq.contiguous(), grad_v_seq.contiguous())
        py_dict.update(ctx.extra)
        if ctx.n_saved > 1:
            py_dict["v_v_seq"] = ctx.saved_tensors[1]
        extra_grads = []
        for name, value in ctx.extra.items():
            if isinstance(value, torch.Tensor):
                py_dict[f"grad_{name}"] = torch.zeros_like(value, dtype=torch.float32)
                extra_grads.append(f"grad_{name}")
        kernel((blocks,), (threads,), py_dict)
        tensor_grads = tuple(py_dict[g] for g in extra_grads)
        return (py_dict["grad_x_seq"], py_dict["grad_v_init"], None, None, None, None, None, *tensor_grads)


def run(x_seq, v_init, v_th, v_reset, forward_kernel, backward_kernel, extra=None):
    if x_seq.dim() != 2 or not x_seq.is_cuda or x_seq.dtype != torch.float32:
        raise ValueError("fragment-assembled kernels take a CUDA float32 tensor of shape [T, N]")
    extra = dict(extra or {})
    tensors = tuple(v for v in extra.values() if isinstance(v, torch.Tensor))
    return KernelPairFunction.apply(x_seq.contiguous(), v_init.contiguous(), float(v_th), None if v_reset is None else float(v_reset),
                                    forward_kernel, backward_kernel, extra, *tensors)
