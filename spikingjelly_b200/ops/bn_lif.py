"""BatchNorm + multi-step neuron as one differentiable op on channels-last activations.

``bn_lif(y, bn, spec, residual=None)`` takes the pre-normalisation tensor ``y``
``[T, ..., C]`` (e.g. a GEMM output), computes batch statistics (or uses the running ones
when ``bn`` is in eval mode), and returns ``LIF_T(BN(y)) (+ residual)`` without ever writing
the normalised tensor.  Backward is two kernels (BPTT + per-channel sums, then the BN
backward in closed form)."""
from __future__ import annotations

from typing import Optional

import torch

from . import counters, require
from .neuron_scan import NeuronSpec

__all__ = ["bn_lif", "BNLIFFunction"]


def _discarded_forward() -> bool:
    """True during the first (thrown-away) forward of a gradient-checkpointed segment
    (``memopt.checkpointing.in_gc_1st_forward``): running statistics are then left alone, exactly like
    ``layer.BatchNorm*`` do, so that only the forward that counts updates them."""
    from ..activation_based.memopt.checkpointing import in_gc_1st_forward
    return in_gc_1st_forward()


class BNLIFFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, gamma, beta, running_mean, running_var, residual, training: bool, momentum: float,
                eps: float, spec: NeuronSpec, v_init: float, need_grad: bool, stats=None):
        vr = 0.0 if spec.soft else float(spec.v_reset)
        if training and stats is not None:
            # the producer (GEMM epilogue) already summed y and y^2 per channel: only the finalisation runs
            counters.bump("bn_stats", 1)
            mean, invstd, scale, shift = torch.ops.sjb200.bn_coefficients_partial(
                stats, y.numel() // y.shape[-1], gamma, beta, running_mean, running_var, momentum, eps)
        else:
            counters.bump("bn_stats", 2 if training else 1)
            mean, invstd, scale, shift = torch.ops.sjb200.bn_coefficients(
                y, gamma, beta, running_mean, running_var, training, momentum, eps)
        counters.bump("bn_lif_forward")
        out, ckpt = torch.ops.sjb200.bn_lif_forward(y, scale, shift, residual, spec.kind, spec.tau, spec.v_threshold,
                                                    vr, spec.soft, v_init, need_grad)
        ctx.spec, ctx.training, ctx.v_init = spec, training, v_init
        ctx.has_residual = residual is not None
        ctx.has_affine = gamma is not None
        ctx.save_for_backward(y, scale, shift, mean, invstd, gamma if gamma is not None else y.new_empty(0), ckpt)
        ctx.mark_dirty()  # running stats are updated through the op's mutable arguments
        return out

    @staticmethod
    def backward(ctx, g_out):
        y, scale, shift, mean, invstd, gamma, ckpt = ctx.saved_tensors
        spec: NeuronSpec = ctx.spec
        vr = 0.0 if spec.soft else float(spec.v_reset)
        counters.bump("bn_lif_backward", 3)
        dy, g_gamma, g_beta = torch.ops.sjb200.bn_lif_backward(
            g_out, y, scale, shift, mean, invstd, gamma if ctx.has_affine else None,
            ckpt if ckpt.numel() > 0 else None, ctx.training, spec.kind, spec.tau, spec.v_threshold, vr, spec.soft,
            ctx.v_init, spec.sg[0], spec.sg[1], spec.sg[2], spec.detach_reset)
        return (dy, g_gamma if ctx.has_affine else None, g_beta if ctx.has_affine else None, None, None,
                g_out if ctx.has_residual else None, None, None, None, None, None, None, None)


def bn_lif(y: torch.Tensor, bn: torch.nn.modules.batchnorm._BatchNorm, spec: NeuronSpec,
           residual: Optional[torch.Tensor] = None, v_init: float = 0.0,
           stats: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y``: contiguous ``[T, ..., C]`` with ``C == bn.num_features`` (channels last).  ``stats``: optional
    ``[blocks, 2, C]`` fp32 partial sums of ``y`` and ``y^2`` per channel (``ops.gemm.linear_with_stats``)."""
    require()
    training, momentum, rm, rv = _bn_args(bn)
    need_grad = torch.is_grad_enabled() and (y.requires_grad or (bn.weight is not None and bn.weight.requires_grad))
    return BNLIFFunction.apply(y.contiguous(), bn.weight, bn.bias, rm, rv, residual, training, momentum, float(bn.eps),
                               spec, float(v_init), need_grad, stats)


class BNPoolLIFFunction(torch.autograd.Function):
    """``LIF_T(maxpool3x3s2(BN(y)))`` on an NHWC conv output (see ``csrc/bn_pool_lif.cu``)."""

    @staticmethod
    def forward(ctx, y, gamma, beta, running_mean, running_var, training: bool, momentum: float, eps: float,
                spec: NeuronSpec, v_init: float, T: int, is_static: bool):
        vr = 0.0 if spec.soft else float(spec.v_reset)
        counters.bump("bn_stats", 2 if training else 1)
        mean, invstd, scale, shift = torch.ops.sjb200.bn_coefficients(
            y, gamma, beta, running_mean, running_var, training, momentum, eps)
        counters.bump("bn_pool_lif_forward")
        out, idx = torch.ops.sjb200.bn_pool_lif_forward(y, scale, shift, T, is_static, spec.kind, spec.tau,
                                                        spec.v_threshold, vr, spec.soft, v_init)
        ctx.spec, ctx.training, ctx.v_init, ctx.T, ctx.is_static = spec, training, v_init, T, is_static
        ctx.has_affine = gamma is not None
        ctx.save_for_backward(y, idx, scale, shift, mean, invstd, gamma if gamma is not None else y.new_empty(0))
        return out

    @staticmethod
    def backward(ctx, g_out):
        y, idx, scale, shift, mean, invstd, gamma = ctx.saved_tensors
        spec: NeuronSpec = ctx.spec
        vr = 0.0 if spec.soft else float(spec.v_reset)
        counters.bump("bn_pool_lif_backward", 3)
        dy, g_gamma, g_beta = torch.ops.sjb200.bn_pool_lif_backward(
            g_out, y, idx, scale, shift, mean, invstd, gamma if ctx.has_affine else None, ctx.training, ctx.T,
            ctx.is_static, spec.kind, spec.tau, spec.v_threshold, vr, spec.soft, ctx.v_init, spec.sg[0], spec.sg[1],
            spec.sg[2], spec.detach_reset)
        return (dy, g_gamma if ctx.has_affine else None, g_beta if ctx.has_affine else None) + (None,) * 9


def _bn_args(bn):
    """``(training, momentum, running_mean, running_var)`` for the statistics kernels; the running tensors are passed
    (and updated in place) only by a training forward that counts."""
    training = bn.training or bn.running_mean is None
    momentum = 0.0 if bn.momentum is None else float(bn.momentum)
    update = bn.training and bn.track_running_stats and not _discarded_forward()
    if update and bn.num_batches_tracked is not None:
        bn.num_batches_tracked.add_(1)
        if bn.momentum is None:
            momentum = 1.0 / float(bn.num_batches_tracked)
    use_running = update or not training
    return training, momentum, (bn.running_mean if use_running else None), (bn.running_var if use_running else None)


def bn_pool_lif(y_nhwc: torch.Tensor, bn, spec: NeuronSpec, T: int, is_static: bool, v_init: float = 0.0):
    """``y_nhwc``: contiguous ``[NB, H, W, C]`` (``NB = B`` when ``is_static`` else ``T*B``), 16-bit.
    Returns spikes ``[T, B, OH, OW, C]`` with ``OH = (H - 1) // 2 + 1``."""
    require()
    training, momentum, rm, rv = _bn_args(bn)
    return BNPoolLIFFunction.apply(y_nhwc, bn.weight, bn.bias, rm, rv, training, momentum, float(bn.eps), spec,
                                   float(v_init), int(T), bool(is_static))
