"""Python front end of the fused multi-step neuron kernels.

``multistep_neuron`` runs charge/fire/reset over the whole sequence in one kernel
and registers a BPTT backward that is one kernel as well.  No intermediate is
saved: backward recomputes the membrane trajectory from ``x_seq`` (plus fp32
checkpoints every ``scan_chunk(T)`` steps when ``T`` is longer than one chunk).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import counters, require

__all__ = ["NeuronSpec", "multistep_neuron", "KIND"]

KIND = {"if": 0, "lif_di": 1, "lif_ndi": 2, "plif_di": 3, "plif_ndi": 4, "qif": 5, "eif": 6}


@dataclass(frozen=True)
class NeuronSpec:
    """Everything the kernel needs to know about the neuron model."""
    kind: int
    v_threshold: float
    v_reset: Optional[float]            # None = soft reset
    tau: float = 2.0
    q: Tuple[float, float, float] = (0.0, 0.0, 0.0)
    sg: Tuple[int, float, float] = (0, 4.0, 0.0)   # surrogate (id, p0, p1)
    detach_reset: bool = False

    @property
    def soft(self) -> bool:
        return self.v_reset is None


class _Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_seq, v_init, r, spec: NeuronSpec, v_init_scalar: float, store_v_seq: bool, pack_bits: bool,
                need_grad: bool, storage_dtype=None):
        vr = 0.0 if spec.soft else float(spec.v_reset)
        ctx.in_dtype = x_seq.dtype
        if storage_dtype is not None and storage_dtype != x_seq.dtype:
            # narrower storage of the input (fp8): cast here, inside the function, so that autograd never sees an fp8
            # tensor (it would round the returned gradient to the input's fp8 dtype)
            x_seq = x_seq.to(storage_dtype)
        counters.bump("scan_forward")
        spike, v_last, v_seq, packed, ckpt = torch.ops.sjb200.scan_forward(
            x_seq, v_init, v_init_scalar, r, spec.kind, spec.tau, spec.q[0], spec.q[1], spec.q[2],
            spec.v_threshold, vr, spec.soft, store_v_seq, pack_bits, need_grad)
        ctx.spec = spec
        ctx.v_init_scalar = v_init_scalar
        ctx.has_v_init = v_init is not None
        ctx.has_r = r is not None
        ctx.store_v_seq = store_v_seq
        ctx.save_for_backward(x_seq, v_init if v_init is not None else x_seq.new_empty(0),
                              r if r is not None else x_seq.new_empty(0), ckpt)
        ctx.mark_non_differentiable(packed)
        ctx.set_materialize_grads(False)
        return spike, v_last, v_seq, packed

    @staticmethod
    def backward(ctx, g_spike, g_v_last, g_v_seq, _g_packed):
        x_seq, v_init, r, ckpt = ctx.saved_tensors
        spec: NeuronSpec = ctx.spec
        vr = 0.0 if spec.soft else float(spec.v_reset)
        if g_spike is None:
            g_spike = torch.zeros_like(x_seq)
        need_gvi = ctx.has_v_init and ctx.needs_input_grad[1]
        counters.bump("scan_backward")
        gx, gvi, gr = torch.ops.sjb200.scan_backward(
            g_spike, g_v_last, g_v_seq if ctx.store_v_seq else None, x_seq,
            v_init if ctx.has_v_init else None, ctx.v_init_scalar, r if ctx.has_r else None,
            ckpt if ckpt.numel() > 0 else None, spec.kind, spec.tau, spec.q[0], spec.q[1], spec.q[2],
            spec.v_threshold, vr, spec.soft, spec.sg[0], spec.sg[1], spec.sg[2], spec.detach_reset, need_gvi)
        g_r = gr.reshape(r.shape).to(r.dtype) if (ctx.has_r and ctx.needs_input_grad[2]) else None
        if gx.dtype != ctx.in_dtype and ctx.in_dtype.is_floating_point and ctx.in_dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
            gx = gx.to(ctx.in_dtype)
        return gx, (gvi if need_gvi else None), g_r, None, None, None, None, None, None


def multistep_neuron(x_seq: torch.Tensor, v_init, spec: NeuronSpec, r: Optional[torch.Tensor] = None,
                     store_v_seq: bool = False, pack_bits: bool = False, storage_dtype: Optional[torch.dtype] = None):
    """Run ``T = x_seq.shape[0]`` steps.  ``v_init`` is a tensor shaped like
    ``x_seq[0]`` or a Python float (uniform initial potential, no memory read).

    Returns ``(spike_seq, v_last, v_seq | None, packed | None)`` where ``packed`` is an
    int32 tensor ``[T, ceil(N/32)]``: bit ``i`` of word ``j`` is neuron ``32 j + i``.  ``storage_dtype`` (fp8 e4m3 / e5m2):
    the input is rounded to that type and kept for backward in it (1 byte per element); spikes and gradients are then bf16
    and the gradient comes back in ``x_seq``'s own dtype.
    """
    require()
    if isinstance(v_init, torch.Tensor):
        v_t, v_s = v_init, 0.0
    else:
        v_t, v_s = None, float(v_init)
    # grad mode is off inside Function.forward, so decide here whether backward can happen
    need_grad = torch.is_grad_enabled() and (
        x_seq.requires_grad or (v_t is not None and v_t.requires_grad) or (r is not None and r.requires_grad))
    spike, v_last, v_seq, packed = _Scan.apply(x_seq, v_t, r, spec, v_s, store_v_seq, pack_bits, need_grad, storage_dtype)
    return spike, v_last, (v_seq if store_v_seq else None), (packed if pack_bits else None)
