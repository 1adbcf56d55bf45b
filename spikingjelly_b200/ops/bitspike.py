"""Spike tensors that exist only as bits.

``multistep_neuron_bits`` runs the fused neuron scan (``ops/csrc/neuron_scan.cuh``) with the dense spike output switched
off: the kernel writes 1 bit per neuron and step (``[T, ceil(N / 32)]`` int32 words, bit ``i`` of word ``j`` = neuron
``32 j + i``) and nothing else, so the forward traffic of a 16-bit layer drops from ``2 + 2`` to ``2 + 1/8`` bytes per
element.  The result is a :class:`BitSpikes`: the words plus a zero-storage *handle* tensor of the logical shape through
which autograd routes the gradient with respect to the spikes.  Consumers:

* :meth:`BitSpikes.dense` - the ordinary 0 / 1 tensor (bit-unpack kernel), differentiable;
* :func:`bit_linear`      - ``spikes @ W^T + b`` that expands the bits right before the tensor-core GEMM and keeps only the
  bits for backward (weight gradient from the re-expanded bits, data gradient straight into the handle).

Backward of the neuron is the usual recomputing scan kernel: it needs the input sequence and the dense gradient with
respect to the spikes, never the spikes themselves."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import counters, require
from .neuron_scan import NeuronSpec

__all__ = ["BitSpikes", "multistep_neuron_bits", "bit_linear"]


@dataclass
class BitSpikes:
    """``words``: int32 ``[T, ceil(N / 32)]``; ``handle``: a float tensor of shape ``shape`` without storage of its own
    (every element aliases one scalar) that carries ``requires_grad``; ``dtype``: the dtype a dense version would have."""
    words: torch.Tensor
    handle: torch.Tensor
    shape: Tuple[int, ...]
    dtype: torch.dtype

    @property
    def nbytes(self) -> int:
        return self.words.numel() * 4

    def dense(self) -> torch.Tensor:
        """The 0 / 1 tensor of shape ``shape``; gradients flow back to the producing neuron."""
        return _Dense.apply(self.handle, self.words, self.shape, self.dtype)


def _unpack(words: torch.Tensor, shape, dtype) -> torch.Tensor:
    T = shape[0]
    n = 1
    for s in shape[1:]:
        n *= s
    if n % 32 == 0:
        flat = torch.ops.sjb200.bit_unpack(words.view(torch.uint8).reshape(-1), T * n, dtype)
        return flat.view(shape)
    rows = [torch.ops.sjb200.bit_unpack(words[t].view(torch.uint8).reshape(-1), n, dtype) for t in range(T)]      # rows are padded to words
    return torch.stack(rows).view(shape)


class _Dense(torch.autograd.Function):
    @staticmethod
    def forward(ctx, handle, words, shape, dtype):
        counters.bump("bit_unpack")
        return _unpack(words, shape, dtype)

    @staticmethod
    def backward(ctx, g):
        return g, None, None, None


class _ScanBits(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_seq, v_init, r, spec: NeuronSpec, v_init_scalar: float, need_grad: bool):
        vr = 0.0 if spec.soft else float(spec.v_reset)
        counters.bump("scan_forward")
        _, v_last, _, packed, ckpt = torch.ops.sjb200.scan_forward(
            x_seq, v_init, v_init_scalar, r, spec.kind, spec.tau, spec.q[0], spec.q[1], spec.q[2], spec.v_threshold, vr, spec.soft,
            False, True, need_grad, True)
        ctx.spec, ctx.v_init_scalar, ctx.has_v_init, ctx.has_r = spec, v_init_scalar, v_init is not None, r is not None
        ctx.save_for_backward(x_seq, v_init if v_init is not None else x_seq.new_empty(0), r if r is not None else x_seq.new_empty(0), ckpt)
        ctx.mark_non_differentiable(packed)
        ctx.set_materialize_grads(False)
        handle = x_seq.new_zeros((), dtype=v_last.dtype).expand(x_seq.shape)
        return handle, v_last, packed

    @staticmethod
    def backward(ctx, g_spike, g_v_last, _g_packed):
        x_seq, v_init, r, ckpt = ctx.saved_tensors
        spec: NeuronSpec = ctx.spec
        vr = 0.0 if spec.soft else float(spec.v_reset)
        if g_spike is None:
            g_spike = torch.zeros_like(x_seq)
        need_gvi = ctx.has_v_init and ctx.needs_input_grad[1]
        counters.bump("scan_backward")
        gx, gvi, gr = torch.ops.sjb200.scan_backward(
            g_spike.contiguous(), g_v_last, None, x_seq, v_init if ctx.has_v_init else None, ctx.v_init_scalar, r if ctx.has_r else None,
            ckpt if ckpt.numel() > 0 else None, spec.kind, spec.tau, spec.q[0], spec.q[1], spec.q[2], spec.v_threshold, vr, spec.soft,
            spec.sg[0], spec.sg[1], spec.sg[2], spec.detach_reset, need_gvi)
        g_r = gr.reshape(r.shape).to(r.dtype) if (ctx.has_r and ctx.needs_input_grad[2]) else None
        return gx, (gvi if need_gvi else None), g_r, None, None, None


def multistep_neuron_bits(x_seq: torch.Tensor, v_init, spec: NeuronSpec, r: Optional[torch.Tensor] = None):
    """``(BitSpikes, v_last)`` of ``T = x_seq.shape[0]`` steps; arguments as in :func:`ops.neuron_scan.multistep_neuron`."""
    require()
    v_t, v_s = (v_init, 0.0) if isinstance(v_init, torch.Tensor) else (None, float(v_init))
    need_grad = torch.is_grad_enabled() and (x_seq.requires_grad or (v_t is not None and v_t.requires_grad) or (r is not None and r.requires_grad))
    handle, v_last, packed = _ScanBits.apply(x_seq, v_t, r, spec, v_s, need_grad)
    return BitSpikes(packed, handle, tuple(x_seq.shape), v_last.dtype), v_last


class _BitLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, handle, words, weight, bias, shape, dtype):
        from . import gemm as G
        x2d = _unpack(words, shape, dtype).reshape(-1, shape[-1])
        w = weight.detach().to(dtype).contiguous()
        y = G.gemm(x2d, w)
        if bias is not None:
            y = y + bias.detach().to(dtype)
        ctx.save_for_backward(words, w)
        ctx.meta = (shape, dtype, weight.dtype, None if bias is None else bias.dtype)
        return y.view(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        from . import gemm as G
        words, w = ctx.saved_tensors
        shape, dtype, wdtype, bdtype = ctx.meta
        g2d = gy.to(dtype).reshape(-1, gy.shape[-1]).contiguous()
        gh = G.gemm(g2d, w, False, True).view(shape) if ctx.needs_input_grad[0] else None
        gw = gb = None
        if ctx.needs_input_grad[2]:
            x2d = _unpack(words, shape, dtype).reshape(-1, shape[-1])
            gw = G.gemm(g2d, x2d, True, True, out_f32=True).to(wdtype)
        if bdtype is not None and ctx.needs_input_grad[3]:
            gb = g2d.sum(0, dtype=torch.float32).to(bdtype)
        return gh, None, gw, gb, None, None


def bit_linear(spikes: BitSpikes, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``F.linear`` on bit-only spikes (16-bit dtypes; feature counts multiples of 8)."""
    require()
    return _BitLinear.apply(spikes.handle, spikes.words, weight, bias, spikes.shape, spikes.dtype)
