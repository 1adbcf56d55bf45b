"""Autograd function around a single-step kernel pair."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..... import configure


class StepPairFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, v, v_th: float, v_reset: Optional[float], forward_kernel, backward_kernel, extra: Dict):
        shape = x.shape
        xf, vf = x.contiguous().view(-1), v.contiguous().view(-1)
        out = torch.empty((3, xf.numel()), device=x.device, dtype=x.dtype)
        py_dict = {"numel": xf.numel(), "x": xf, "v": vf, "h": out[0], "spike": out[1], "v_next": out[2], "v_th": v_th, **extra}
        if v_reset is not None:
            py_dict["v_reset"] = v_reset
        threads = configure.cuda_threads
        blocks = (xf.numel() + threads - 1) // threads
        forward_kernel((blocks,), (threads,), py_dict)
        if x.requires_grad or v.requires_grad:
            ctx.save_for_backward(out[0])
            ctx.meta = (v_th, v_reset, backward_kernel, extra, blocks, threads, shape)
        return out[1].view(shape), out[2].view(shape)

    @staticmethod
    def backward(ctx, grad_spike, grad_v_next):
        v_th, v_reset, kernel, extra, blocks, threads, shape = ctx.meta
        (h,) = ctx.saved_tensors
        grads = torch.empty((2, h.numel()), device=h.device, dtype=h.dtype)
        py_dict = {"numel": h.numel(), "grad_spike": grad_spike.contiguous().view(-1), "grad_v_next": grad_v_next.contiguous().view(-1), "h": h,
                   "grad_x": grads[0], "grad_v": grads[1], "v_th": v_th, **extra}
        if v_reset is not None:
            py_dict["v_reset"] = v_reset
        kernel((blocks,), (threads,), py_dict)
        return grads[0].view(shape), grads[1].view(shape), None, None, None, None, None


def run(x, v, v_th, v_reset, forward_kernel, backward_kernel, extra=None):
    if not x.is_cuda or x.dtype != torch.float32:
        raise ValueError("fragment-assembled kernels take CUDA float32 tensors")
    return StepPairFunction.apply(x, v, float(v_th), None if v_reset is None else float(v_reset), forward_kernel, backward_kernel, dict(extra or {}))
