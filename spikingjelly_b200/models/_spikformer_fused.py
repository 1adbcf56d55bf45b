"""Fused channels-last execution of :class:`Spikformer` on CUDA.

Same parameters, same mathematics as the module-by-module forward, different schedule:

* activations are channels-last (``[T, B, L, C]`` tokens / NHWC feature maps), so every
  1x1 convolution is one row-major GEMM over ``M = T*B*L`` rows on the tcgen05 kernel;
* every ``BatchNorm -> LIF`` pair (and the residual add that follows it) is one fused
  op (:func:`spikingjelly_b200.ops.bn_lif.bn_lif`): the normalised tensor is never stored;
* a static image input is identical at every time step, so the first stem stage
  (conv, BN statistics, max-pool) is evaluated once on ``B`` images and only the neuron
  runs over ``T`` — its backward sums the per-step gradients, which is exactly what the
  repeated computation would produce.

The fused path assumes that all neurons start from their reset state (the usual
``forward -> backward -> reset_net`` training step) and does not materialise membrane
potentials; it is skipped (module path used instead) whenever that does not hold.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..activation_based import base, neuron, surrogate
from ..ops import conv as conv_ops
from ..ops import conv_stem as stem_ops
from ..ops import gemm as G
from ..ops.bn_lif import bn_lif, bn_pool_lif
from ..ops.ssa import ssa as ssa_op
from ..ops.neuron_scan import KIND, NeuronSpec, multistep_neuron

__all__ = ["forward", "eligible"]


def _spec(lif: neuron.LIFNode) -> Optional[NeuronSpec]:
    sg = surrogate.surrogate_spec(lif.surrogate_function)
    if sg is None or not isinstance(lif, neuron.LIFNode):
        return None
    return NeuronSpec(KIND["lif_di" if lif.decay_input else "lif_ndi"], float(lif.v_threshold),
                      None if lif.v_reset is None else float(lif.v_reset), float(lif.tau), (0.0, 0.0, 0.0), sg,
                      bool(lif.detach_reset))


def _compute_dtype(x: torch.Tensor) -> Optional[torch.dtype]:
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        return dt if dt in (torch.bfloat16, torch.float16) else None
    return x.dtype if x.dtype in (torch.bfloat16, torch.float16) else None


def eligible(model, x: torch.Tensor) -> bool:
    """True when the fused schedule reproduces the module path for this call."""
    if not x.is_cuda or _compute_dtype(x) is None or x.ndim not in (4, 5):
        return False
    if model.embed_dims % 64 != 0 or (model.embed_dims // model.num_heads) % 8 != 0:
        return False
    for m in model.modules():
        if isinstance(m, neuron.BaseNode):
            if not isinstance(m, neuron.LIFNode) or not isinstance(m._memories.get("v"), float) or m.store_v_seq:
                return False
            if _spec(m) is None or not m.native:
                return False
            if m._memories["v"] != (m.v_reset if m.v_reset is not None else 0.0):
                return False
        elif isinstance(m, nn.modules.batchnorm._BatchNorm) and (not m.affine or isinstance(m, nn.SyncBatchNorm)):
            return False        # SyncBatchNorm needs statistics over all ranks; the fused kernels keep them per process
    return True


def _init_v(lif) -> float:
    return float(lif.v_reset) if lif.v_reset is not None else 0.0


def _stem_stage(stage, h: torch.Tensor, T: int, static: bool, dt) -> torch.Tensor:
    """``h``: NHWC-in-memory ``[T*B (or B when static), C, H, W]`` -> spikes ``[T*B, C', H', W']``."""
    conv, bn = stage.conv_bn.block[0], stage.conv_bn.block[1]
    pool = stage.conv_bn.block[2] if len(stage.conv_bn.block) > 2 else None
    if stem_ops.supports(conv, h):
        # the image itself (3 channels): patch matrix + tensor-core GEMM instead of cuDNN's padded-channel kernel
        rows, _, (oh, ow) = stem_ops.conv2d_few_channels(h, conv.weight, conv.stride, conv.padding, want_stats=False)
        y = rows.view(h.shape[0], oh, ow, rows.shape[1]).permute(0, 3, 1, 2)
    elif conv_ops.supports(conv, h) and conv.bias is None:
        # implicit GEMM on the tensor cores (TMA-gathered patches), output rows are the channels-last result
        rows, _, (oh, ow) = conv_ops.conv2d_rows(h.permute(0, 2, 3, 1), conv.weight, conv.stride, conv.padding, conv.dilation)
        y = rows.view(h.shape[0], oh, ow, rows.shape[1]).permute(0, 3, 1, 2)
    else:
        y = F.conv2d(h, conv.weight.to(dt), None if conv.bias is None else conv.bias.to(dt), conv.stride, conv.padding,
                     conv.dilation, conv.groups)
    lif = stage.neuron
    spec = _spec(lif)
    if pool is None:
        # [T*B, C, H, W] channels-last == [T, B*H*W, C] row-major
        n, c, hh, ww = y.shape
        rows = y.permute(0, 2, 3, 1).reshape(T, (n // T) * hh * ww, c)
        res = h.permute(0, 2, 3, 1).reshape(T, (n // T) * hh * ww, c)
        out = bn_lif(rows, bn, spec, residual=res, v_init=_init_v(lif))
        return out.reshape(n, hh, ww, c).permute(0, 3, 1, 2)
    if (pool.kernel_size, pool.stride, pool.padding) in ((3, 2, 1), ((3, 3), (2, 2), (1, 1))) and T <= 8:
        n, c, hh, ww = y.shape
        out = bn_pool_lif(y.permute(0, 2, 3, 1), bn, spec, T, static, v_init=_init_v(lif))   # [T, B, OH, OW, C]
        return out.flatten(0, 1).permute(0, 3, 1, 2)
    z = F.batch_norm(y, bn.running_mean, bn.running_var, bn.weight, bn.bias, bn.training,
                     0.0 if bn.momentum is None else bn.momentum, bn.eps)
    if bn.training and bn.num_batches_tracked is not None:
        bn.num_batches_tracked.add_(1)
    p = F.max_pool2d(z, pool.kernel_size, pool.stride, pool.padding)
    n, c, hh, ww = p.shape
    flat = p.permute(0, 2, 3, 1)
    if static:
        seq = flat.reshape(1, n * hh * ww * c).expand(T, -1)
        b = n
    else:
        seq = flat.reshape(T, (n // T) * hh * ww * c)
        b = n // T
    s, _, _, _ = multistep_neuron(seq, _init_v(lif), spec)
    return s.reshape(T * b, hh, ww, c).permute(0, 3, 1, 2)


def _ssa(S: torch.Tensor, T: int, B: int, L: int, heads: int, scale: float) -> torch.Tensor:
    """``S``: spikes ``[T, B*L, 3C]`` -> ``Q (K^T V) * scale`` as ``[T, B*L, C]``."""
    C = S.shape[-1] // 3
    d = C // heads
    if d in (32, 64) and (4 * ((L + 15) // 16 * 16) + 2 * d) * (d + 8) * 2 <= 220 * 1024:
        return ssa_op(S, L, heads, scale)
    qkv = S.view(T, B, L, 3, heads, d)
    q, k, v = qkv.unbind(3)
    kv = torch.einsum("tblhd,tblhe->tbhde", k, v)
    out = torch.einsum("tblhd,tbhde->tblhe", q, kv) * scale
    return out.reshape(T, B * L, C)


def _linear_bn(x2d: torch.Tensor, w: torch.Tensor, bn):
    """The token GEMM; in training mode its epilogue also emits the per-channel sums the batch norm needs."""
    if bn.training or bn.running_mean is None:
        return G.linear_with_stats(x2d, w)
    return G.linear(x2d, w), None


def _block(blk, X: torch.Tensor, T: int, B: int, L: int, dt) -> torch.Tensor:
    """``X``: ``[T, B*L, C]`` contiguous tokens."""
    C = X.shape[-1]
    M = T * B * L
    attn, mlp = blk.attn, blk.mlp
    w_qkv = attn.qkv_conv_bn[0].weight.squeeze(-1).to(dt)
    y, st = _linear_bn(X.view(M, C), w_qkv, attn.qkv_conv_bn[1])
    S = bn_lif(y.view(T, B * L, 3 * C), attn.qkv_conv_bn[1], _spec(attn.qkv_lif), v_init=_init_v(attn.qkv_lif), stats=st)
    a = _ssa(S, T, B, L, attn.num_heads, attn.scale)
    A, _, _, _ = multistep_neuron(a.reshape(T, -1), _init_v(attn.attn_lif), _spec(attn.attn_lif))
    w_proj = attn.proj_conv_bn[0].weight.squeeze(-1).to(dt)
    y, st = _linear_bn(A.view(M, C), w_proj, attn.proj_conv_bn[1])
    X1 = bn_lif(y.view(T, B * L, C), attn.proj_conv_bn[1], _spec(attn.proj_lif), residual=X, v_init=_init_v(attn.proj_lif), stats=st)
    w1 = mlp.fc1[0].weight.squeeze(-1).to(dt)
    y, st = _linear_bn(X1.view(M, C), w1, mlp.fc1[1])
    F1 = bn_lif(y.view(T, B * L, -1), mlp.fc1[1], _spec(mlp.neuron1), v_init=_init_v(mlp.neuron1), stats=st)
    w2 = mlp.fc2[0].weight.squeeze(-1).to(dt)
    y, st = _linear_bn(F1.view(M, F1.shape[-1]), w2, mlp.fc2[1])
    return bn_lif(y.view(T, B * L, C), mlp.fc2[1], _spec(mlp.neuron2), residual=X1, v_init=_init_v(mlp.neuron2), stats=st)


def forward(model, x: torch.Tensor) -> torch.Tensor:
    dt = _compute_dtype(x)
    T = model.T if x.ndim == 4 else x.shape[0]
    static = x.ndim == 4
    with torch.autocast("cuda", enabled=False):
        if static:
            B = x.shape[0]
            h = x.to(dt).contiguous(memory_format=torch.channels_last)
        else:
            B = x.shape[1]
            h = x.flatten(0, 1).to(dt).contiguous(memory_format=torch.channels_last)
        stem = model.patch_embed
        for i, stage in enumerate(stem.stages):
            h = _stem_stage(stage, h, T, static and i == 0, dt)
        h = _stem_stage(stem.positional_encoding, h, T, False, dt)      # includes the residual add
        n, C, hh, ww = h.shape
        L = hh * ww
        X = h.permute(0, 2, 3, 1).reshape(T, B * L, C)
        for blk in model.blocks:
            X = _block(blk, X, T, B, L, dt)
        base.elide_states(m for m in model.modules() if isinstance(m, neuron.BaseNode))
        feat = X.view(T, B, L, C).mean(dim=2)
        return F.linear(feat, model.head.weight.to(dt), None if model.head.bias is None else model.head.bias.to(dt))
