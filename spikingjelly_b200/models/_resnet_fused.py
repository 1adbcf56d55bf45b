"""Fused execution schedule of the SEW-ResNet family on B200.

The module path runs every stage as convolution (cuDNN) -> BatchNorm (three library kernels forward, one large one
backward) -> neuron kernel, on NCHW tensors that cuDNN converts to NHWC and back around each convolution.  Here the
whole trunk stays channels-last: a convolution's output ``[T*B, H, W, C]`` is handed as rows ``[T, B*H*W, C]`` to the
fused BatchNorm+LIF kernels (``ops/csrc/bn_lif.cu``: batch statistics, then BN applied inside the LIF scan; backward =
BPTT + closed-form BN backward), which also add the SEW shortcut (``cnf="ADD"``) on the way out.  Nothing but the
convolution output and the spikes ever exists in memory, and no layout conversion is left.

Used automatically by :class:`~spikingjelly_b200.models._resnet_family.ResidualSNN` when :func:`eligible` holds
(CUDA input, 16-bit compute, multi-step mode, native LIF / IF neurons in their reset state, affine BatchNorm2d);
results equal the module path up to the rounding points of 16-bit arithmetic.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..activation_based import base, layer, neuron, surrogate
from ..ops import conv as conv_ops
from ..ops import conv_stem as stem_ops
from ..ops import pool as pool_ops
from ..ops.bn_lif import bn_lif
from ..ops.neuron_scan import KIND, NeuronSpec

__all__ = ["eligible", "forward"]


def _spec(n) -> Optional[NeuronSpec]:
    sg = surrogate.surrogate_spec(n.surrogate_function)
    if sg is None:
        return None
    v_reset = None if n.v_reset is None else float(n.v_reset)
    if type(n) is neuron.LIFNode:
        return NeuronSpec(KIND["lif_di" if n.decay_input else "lif_ndi"], float(n.v_threshold), v_reset, float(n.tau), (0.0, 0.0, 0.0), sg,
                          bool(n.detach_reset))
    if type(n) is neuron.IFNode:
        return NeuronSpec(KIND["if"], float(n.v_threshold), v_reset, 2.0, (0.0, 0.0, 0.0), sg, bool(n.detach_reset))
    return None


def _compute_dtype(x: torch.Tensor) -> Optional[torch.dtype]:
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        return dt if dt in (torch.bfloat16, torch.float16) else None
    return x.dtype if x.dtype in (torch.bfloat16, torch.float16) else None


def bn_is_fusable(m) -> bool:
    """Plain affine BatchNorm2d with per-process statistics.  SyncBatchNorm needs statistics over all ranks, which the
    fused kernels do not exchange."""
    return isinstance(m, nn.BatchNorm2d) and not isinstance(m, nn.SyncBatchNorm) and m.affine and m.num_features % 8 == 0


def eligible(model, x: torch.Tensor) -> bool:
    if not x.is_cuda or x.ndim != 5 or _compute_dtype(x) is None:
        return False
    if not all(getattr(blk, "sew", False) for stage in (model.layer1, model.layer2, model.layer3, model.layer4) for blk in stage):
        return False
    if not isinstance(model.maxpool, layer.MaxPool2d) or model.maxpool.step_mode != "m":
        return False
    for m in model.modules():
        if isinstance(m, neuron.BaseNode):
            if _spec(m) is None or not m.native or m.step_mode != "m" or m.store_v_seq or not isinstance(m._memories.get("v"), float):
                return False
            if m._memories["v"] != (m.v_reset if m.v_reset is not None else 0.0):
                return False
        elif isinstance(m, nn.modules.batchnorm._BatchNorm):
            if not bn_is_fusable(m):
                return False
        elif isinstance(m, nn.Conv2d) and (m.bias is not None or m.padding_mode != "zeros"):
            return False
    return True


def _init_v(n) -> float:
    return float(n.v_reset) if n.v_reset is not None else 0.0


def _conv(conv: nn.Conv2d, h: torch.Tensor) -> torch.Tensor:
    # the cast to the compute dtype also lays the filter out channels-last, so cuDNN's NHWC kernels take it as it is
    # (the parameter itself keeps its layout: optimizers and gradient buckets rely on it)
    w = conv.weight.to(dtype=h.dtype, memory_format=torch.channels_last)
    return F.conv2d(h, w, None, conv.stride, conv.padding, conv.dilation, conv.groups)


def _rows(t: torch.Tensor, T: int) -> torch.Tensor:
    """NCHW-shaped channels-last tensor -> contiguous ``[T, B*H*W, C]`` view."""
    r = t.permute(0, 2, 3, 1)
    if not r.is_contiguous():
        r = r.contiguous()
    return r.reshape(T, -1, r.shape[-1])


def _stage(conv, bn, sn, h: torch.Tensor, T: int, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    if residual is None and stem_ops.supports(conv, h):
        # few input channels (the network input): patch matrix + tensor-core GEMM whose epilogue also sums the BN statistics
        training = bn.training or bn.running_mean is None
        rows, stats, (H, W) = stem_ops.conv2d_few_channels(h, conv.weight, conv.stride, conv.padding, want_stats=training)
        C = rows.shape[1]
        out = bn_lif(rows.view(T, -1, C), bn, _spec(sn), v_init=_init_v(sn), stats=stats)
        return out.view(h.shape[0], H, W, C).permute(0, 3, 1, 2)
    res_rows = None if residual is None else _rows(residual, T)
    if conv_ops.supports(conv, h):
        # implicit GEMM on the tensor cores; the epilogue sums the BN statistics
        training = bn.training or bn.running_mean is None
        rows, stats, (H, W) = conv_ops.conv2d_rows(h.permute(0, 2, 3, 1), conv.weight, conv.stride, conv.padding, conv.dilation,
                                                   want_stats=training)
        C = rows.shape[1]
        out = bn_lif(rows.view(T, -1, C), bn, _spec(sn), residual=res_rows, v_init=_init_v(sn), stats=stats)
        return out.view(h.shape[0], H, W, C).permute(0, 3, 1, 2)
    y = _conv(conv, h)
    TB, C, H, W = y.shape
    out = bn_lif(_rows(y, T), bn, _spec(sn), residual=res_rows, v_init=_init_v(sn))
    return out.view(TB, H, W, C).permute(0, 3, 1, 2)


def _block(blk, x: torch.Tensor, T: int) -> torch.Tensor:
    identity = x if blk.downsample is None else _stage(blk.downsample[0], blk.downsample[1], blk.downsample_sn, x, T)
    out = x
    stages = blk._stages
    for i, (conv, bn, sn) in enumerate(stages):
        last = i + 1 == len(stages)
        fuse_add = last and blk.cnf == "ADD"
        out = _stage(getattr(blk, conv), getattr(blk, bn), getattr(blk, sn), out, T, residual=identity if fuse_add else None)
    if blk.cnf == "ADD":
        return out
    if blk.cnf == "AND":
        return identity * out
    if blk.cnf == "IAND":
        return identity * (1.0 - out) if blk._identity_first else out * (1.0 - identity)
    raise NotImplementedError(blk.cnf)


def forward(model, x: torch.Tensor) -> torch.Tensor:
    T, B = x.shape[0], x.shape[1]
    dt = _compute_dtype(x)
    h = x.flatten(0, 1).to(dt).contiguous(memory_format=torch.channels_last)
    h = _stage(model.conv1, model.bn1, model.sn1, h, T)
    mp = model.maxpool
    if pool_ops.supports(mp, h):
        h = pool_ops.max_pool_3x3s2_channels_last(h)
    else:
        h = F.max_pool2d(h, mp.kernel_size, mp.stride, mp.padding, mp.dilation, mp.ceil_mode)
    for stage in (model.layer1, model.layer2, model.layer3, model.layer4):
        for blk in stage:
            h = _block(blk, h, T)
    base.elide_states(m for m in model.modules() if isinstance(m, neuron.BaseNode))
    size = model.avgpool.output_size
    size = (size, size) if isinstance(size, int) else tuple(size)
    if size == (1, 1):
        feat = h.float().mean((2, 3)).to(h.dtype).view(T, B, -1)
    else:
        feat = torch.flatten(F.adaptive_avg_pool2d(h, size), 1).view(T, B, -1)
    return model.fc(feat)
