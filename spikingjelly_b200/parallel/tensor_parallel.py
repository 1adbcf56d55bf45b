"""Tensor parallelism on plain process groups (Megatron style), for linear layers, 1x1 / kxk
convolution stacks and Spikformer blocks.

A *column-parallel* layer keeps a slice of the output features (rows of ``weight``); its output is the
local slice (``colwise_local_output``) or is all-gathered (``colwise``).  A *row-parallel* layer keeps a
slice of the input features; it consumes a local slice and all-reduces its partial products.  The
differentiable collectives are ``autograd.Function``s, every all-reduce is counted by the debug
statistics, and the neuron between a column- and a row-parallel layer works on the local slice (its
state is sharded with its input).

Spikes are what crosses ranks in an SNN: the forward all-reduce of a row-parallel layer sums
pre-activations, but the all-gather of a column-parallel output moves {0, 1} values and is sent
bit-packed when the payload is binary (``pack_spikes=True``; 16x less traffic than bf16).

Parity: ``spikingjelly/activation_based/distributed/tensor_parallel/{linear,channel,state,debug,
spikformer,cifar10dvs_vgg}.py`` (the reference builds on DTensor; the public names and styles are kept).
"""
from __future__ import annotations

import copy
import threading
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Sequence, Union

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..activation_based import base, layer
from .analysis import _iter_named_modules_under_roots, analyze_snn_distributed_capability, linear_like_types
from .mesh import _resolve_mesh_dim_group

__all__ = ["TENSOR_PARALLEL_AVAILABLE", "enable_tp_communication_debug", "reset_tp_communication_debug_stats",
           "get_tp_communication_debug_stats", "make_tensor_shard_memory_module", "auto_build_tensor_parallel_plan",
           "wrap_tp_memory_modules", "parallelize_snn_module", "ColwiseParallelLinear", "RowwiseParallelLinear",
           "ChannelShardConv1d", "ChannelShardConv2d", "ChannelShardBatchNorm1d", "ChannelShardBatchNorm2d",
           "parallelize_snn_conv_blocks", "parallelize_spikformer_blocks", "parallelize_spikformer_patch_stem", "TP_STYLES"]

TENSOR_PARALLEL_AVAILABLE = True
TP_STYLES = ("colwise", "colwise_shard", "colwise_local_output", "colwise_local", "rowwise", "td_colwise_replicated",
             "td_rowwise_replicated")

# ------------------------------------------------------------------------------- debug counters
_debug_enabled = False
_debug_stats = {"all_reduce_calls": 0, "all_reduce_bytes": 0, "all_gather_calls": 0, "all_gather_bytes": 0}
_debug_lock = threading.Lock()


def enable_tp_communication_debug(enabled: bool = True) -> None:
    """Switch the counting of tensor-parallel collectives (calls and payload bytes) on or off."""
    global _debug_enabled
    _debug_enabled = bool(enabled)


def reset_tp_communication_debug_stats() -> None:
    with _debug_lock:
        for k in _debug_stats:
            _debug_stats[k] = 0


def get_tp_communication_debug_stats() -> Dict[str, int]:
    with _debug_lock:
        return {k: int(v) for k, v in _debug_stats.items()}


def _record(kind: str, nbytes: int) -> None:
    if _debug_enabled:
        with _debug_lock:
            _debug_stats[f"{kind}_calls"] += 1
            _debug_stats[f"{kind}_bytes"] += int(nbytes)


def _record_tp_all_reduce(t: torch.Tensor) -> None:
    _record("all_reduce", t.numel() * t.element_size())


# ---------------------------------------------------------------------- differentiable collectives
def _ws(group) -> int:
    return dist.get_world_size(group) if (group is not None or dist.is_initialized()) and dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def _all_reduce(t: torch.Tensor, group) -> torch.Tensor:
    if _ws(group) == 1:
        return t
    t = t.contiguous()
    _record_tp_all_reduce(t)
    dist.all_reduce(t, group=group)
    return t


def _all_gather(t: torch.Tensor, group, dim: int, pack_spikes: bool) -> torch.Tensor:
    ws = _ws(group)
    if ws == 1:
        return t
    t = t.contiguous()
    if pack_spikes and not t.requires_grad and t.is_floating_point() and bool(((t == 0) | (t == 1)).all()):
        from ..ops.bitpack import bit_spike_compress, bit_spike_decompress
        packed = bit_spike_compress(t)
        parts = [torch.empty_like(packed) for _ in range(ws)]
        _record("all_gather", packed.numel() * ws)
        dist.all_gather(parts, packed, group=group)
        return torch.cat([bit_spike_decompress(p, t.shape, t.dtype) for p in parts], dim=dim)
    parts = [torch.empty_like(t) for _ in range(ws)]
    _record("all_gather", t.numel() * t.element_size() * ws)
    dist.all_gather(parts, t, group=group)
    return torch.cat(parts, dim=dim)


class _CopyToGroup(torch.autograd.Function):
    """identity forward, all-reduce backward (the input of a column-parallel layer)"""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g.clone(), ctx.group), None


class _ReduceFromGroup(torch.autograd.Function):
    """all-reduce forward, identity backward (the output of a row-parallel layer)"""

    @staticmethod
    def forward(ctx, x, group):
        return _all_reduce(x.clone(), group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherFromGroup(torch.autograd.Function):
    """all-gather along ``dim`` forward, keep the local slice backward"""

    @staticmethod
    def forward(ctx, x, group, dim, pack_spikes):
        ctx.group, ctx.dim, ctx.n = group, dim, x.shape[dim]
        return _all_gather(x.detach(), group, dim, pack_spikes)

    @staticmethod
    def backward(ctx, g):
        r = _rank(ctx.group)
        return g.narrow(ctx.dim, r * ctx.n, ctx.n).contiguous(), None, None, None


class _ScatterToGroup(torch.autograd.Function):
    """keep the local slice forward, all-gather backward"""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        n = x.shape[dim] // _ws(group)
        return x.narrow(dim, _rank(group) * n, n).contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather(g, ctx.group, ctx.dim, False), None, None


def _even(total: int, ws: int, what: str) -> int:
    if total % ws:
        raise ValueError(f"{what}={total} must be divisible by tensor-parallel world_size={ws}.")
    return total // ws


def _shard_param(p: Optional[torch.Tensor], dim: int, group) -> Optional[nn.Parameter]:
    if p is None:
        return None
    n = _even(p.shape[dim], _ws(group), "sharded dimension")
    return nn.Parameter(p.detach().narrow(dim, _rank(group) * n, n).clone(), requires_grad=p.requires_grad)


# ------------------------------------------------------------------------------- linear layers
class ColwiseParallelLinear(nn.Module):
    """``y[..., rows of this rank] = x W_r^T + b_r``.  ``gather_output``: return the full output."""

    def __init__(self, source: nn.Linear, group=None, gather_output: bool = False, pack_spikes: bool = False):
        super().__init__()
        self.group, self.gather_output, self.pack_spikes = group, gather_output, pack_spikes
        self.in_features, self.out_features = source.in_features, source.out_features
        self.weight = _shard_param(source.weight, 0, group)
        self.bias = _shard_param(source.bias, 0, group)
        self.step_mode = getattr(source, "step_mode", "s")

    def forward(self, x):
        ws = _ws(self.group)
        if ws > 1 and x.shape[-1] * ws == self.in_features:       # fed by another column-parallel layer
            x = _GatherFromGroup.apply(x, self.group, x.dim() - 1, self.pack_spikes)
        y = F.linear(_CopyToGroup.apply(x, self.group), self.weight, self.bias)
        return _GatherFromGroup.apply(y, self.group, y.dim() - 1, False) if self.gather_output else y

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features} (local {self.weight.shape[0]}), gather_output={self.gather_output}"


class RowwiseParallelLinear(nn.Module):
    """``y = sum over ranks of x_r W_r^T (+ b)``; takes the local input slice (or slices a full input)."""

    def __init__(self, source: nn.Linear, group=None):
        super().__init__()
        self.group = group
        self.in_features, self.out_features = source.in_features, source.out_features
        self.weight = _shard_param(source.weight, 1, group)
        self.bias = None if source.bias is None else nn.Parameter(source.bias.detach().clone(), requires_grad=source.bias.requires_grad)
        self.step_mode = getattr(source, "step_mode", "s")

    def forward(self, x):
        if x.shape[-1] == self.in_features and _ws(self.group) > 1:
            x = _ScatterToGroup.apply(x, self.group, x.dim() - 1)
        y = _ReduceFromGroup.apply(F.linear(x, self.weight), self.group)
        return y if self.bias is None else y + self.bias

    def extra_repr(self):
        return f"in_features={self.in_features} (local {self.weight.shape[1]}), out_features={self.out_features}"


def _normalize_style(style) -> str:
    if not isinstance(style, str):
        name = type(style).__name__.lower()
        if "rowwise" in name:
            return "rowwise"
        if "colwise" in name:
            return "colwise_local_output" if getattr(style, "use_local_output", False) else "colwise"
        raise ValueError(f"Unsupported tensor parallel style object {style!r}.")
    s = style.lower()
    if s not in TP_STYLES:
        raise ValueError(f"Unsupported tensor parallel style '{style}'. Expected one of: colwise, colwise_local_output, "
                         "rowwise, td_colwise_replicated, td_rowwise_replicated.")
    return {"colwise_shard": "colwise", "colwise_local": "colwise_local_output"}.get(s, s)


def auto_build_tensor_parallel_plan(module: nn.Module, tensor_parallel_roots: Optional[Sequence[str]] = None) -> Dict[str, str]:
    """Every Linear-like candidate becomes column-parallel (local output when there are several),
    the last one row-parallel — a chain ``colwise -> ... -> rowwise`` needs one all-reduce."""
    names = list(analyze_snn_distributed_capability(module, tensor_parallel_roots).tensor_parallel_candidate_names)
    if not names:
        raise ValueError("No Linear-like modules were found for tensor parallelism.")
    plan = {}
    for i, name in enumerate(names):
        rowwise = len(names) > 1 and i == len(names) - 1
        plan[name] = "rowwise" if rowwise else ("colwise_local_output" if len(names) > 1 else "colwise")
    return plan


def _replace(parent: nn.Module, child_name: str, new: nn.Module) -> None:
    if isinstance(parent, (nn.Sequential, nn.ModuleList)) and child_name.isdigit():
        parent[int(child_name)] = new
    else:
        setattr(parent, child_name, new)


def _group_of(device_mesh_or_group, tp_mesh_dim: int):
    if device_mesh_or_group is None:
        return dist.group.WORLD if dist.is_initialized() else None
    if isinstance(device_mesh_or_group, dist.ProcessGroup):
        return device_mesh_or_group
    return _resolve_mesh_dim_group(device_mesh_or_group, tp_mesh_dim)


def parallelize_snn_module(module: nn.Module, device_mesh, tensor_parallel_plan: Mapping[str, Any], tp_mesh_dim: int = 0) -> nn.Module:
    """Replace the planned linear layers by their sharded versions, in place.  ``device_mesh`` may be
    a ``DeviceMesh`` (axis ``tp_mesh_dim`` is used), a process group, or ``None`` (default group)."""
    group = _group_of(device_mesh, tp_mesh_dim)
    named = dict(module.named_modules())
    for name, style in tensor_parallel_plan.items():
        if name not in named:
            raise KeyError(f"tensor_parallel_plan contains unknown module path '{name}'.")
        src = named[name]
        if isinstance(src, (ColwiseParallelLinear, RowwiseParallelLinear)):
            continue
        if not isinstance(src, linear_like_types()):
            raise TypeError(f"'{name}' is a {type(src).__name__}; tensor-parallel styles apply to Linear-like modules.")
        s = _normalize_style(style)
        if s in ("rowwise", "td_rowwise_replicated"):
            new = RowwiseParallelLinear(src, group)
        else:
            new = ColwiseParallelLinear(src, group, gather_output=s in ("colwise", "td_colwise_replicated"))
        parent_name, _, child = name.rpartition(".")
        _replace(named[parent_name] if parent_name else module, child, new)
    return module


# ------------------------------------------------------------------------------ sharded neuron state
_VALIDATOR_ATTR = "_tensor_shard_input_validator"


@dataclass(frozen=True)
class _TensorShardInputValidator:
    shard_dim: int
    logical_dim_size: Optional[int]
    rank: int
    world_size: int
    expected_local_dim_size: Optional[int]

    def __call__(self, _module, args, kwargs) -> None:
        if args:
            x = args[0]
        elif "x" in kwargs:
            x = kwargs["x"]
        else:
            raise TypeError("Shard validation requires the input tensor as the first positional argument or the 'x' keyword argument.")
        d = self.shard_dim if self.shard_dim >= 0 else x.dim() + self.shard_dim
        if d < 0 or d >= x.dim():
            raise ValueError(f"shard_dim={d} (from self.shard_dim={self.shard_dim}) is invalid for input with shape {tuple(x.shape)}.")
        if self.expected_local_dim_size is not None and x.shape[d] != self.expected_local_dim_size:
            raise ValueError(f"Expected local shard size {self.expected_local_dim_size} on dim {d}, but got input shape {tuple(x.shape)}.")


def _has_validator(m) -> bool:
    v = getattr(m, _VALIDATOR_ATTR, None)
    return isinstance(v, _TensorShardInputValidator) and any(h == v for h in m._forward_pre_hooks.values())


def make_tensor_shard_memory_module(source: base.MemoryModule, shard_dim: int, logical_dim_size: Optional[int] = None,
                                    process_group: Optional[Any] = None) -> base.MemoryModule:
    """A copy of a stateful module that is declared to work on the local slice of dimension
    ``shard_dim`` (``logical_dim_size`` = full size): a forward pre-hook checks every input's local
    size, so that a replicated tensor reaching a sharded neuron is an error instead of silently
    wrong state.  Element-wise neurons need nothing else — their state takes the input's shape."""
    if _has_validator(source):
        return source
    m = copy.deepcopy(source)
    step_mode = getattr(m, "step_mode", "s")
    eff_dim = 1 if shard_dim == 2 and step_mode == "s" else shard_dim
    rank = dist.get_rank(process_group) if process_group is not None else 0
    ws = dist.get_world_size(process_group) if process_group is not None else 1
    local = None if logical_dim_size is None else _even(logical_dim_size, ws, "logical_dim_size")
    v = _TensorShardInputValidator(eff_dim, logical_dim_size, rank, ws, local)
    m.register_forward_pre_hook(v, with_kwargs=True)
    setattr(m, _VALIDATOR_ATTR, v)
    return m


def wrap_tp_memory_modules(module: nn.Module, tensor_parallel_plan: Mapping[str, Any], process_group):
    """Inside ``nn.Sequential`` / ``nn.ModuleList`` parents: the stateful module that follows a
    ``colwise_local_output`` linear layer (skipping Dropout / Identity) is marked as sharded."""
    named = dict(module.named_modules())
    for name, style in tensor_parallel_plan.items():
        if _normalize_style(style) != "colwise_local_output":
            continue
        src = named.get(name)
        if not isinstance(src, linear_like_types()):
            continue
        parent_name, _, child = name.rpartition(".")
        parent = module if not parent_name else named[parent_name]
        if not isinstance(parent, (nn.Sequential, nn.ModuleList)) or not child.isdigit():
            continue
        i = int(child) + 1
        while i < len(parent) and isinstance(parent[i], (nn.Dropout, nn.Identity, layer.Dropout)):
            i += 1
        if i < len(parent) and isinstance(parent[i], base.MemoryModule):
            parent[i] = make_tensor_shard_memory_module(parent[i], -1, src.out_features, process_group)
    return module


# ------------------------------------------------------------------------- channel-sharded convolutions
class _ChannelShardConv(nn.Module):
    """Convolution sharded over channels.  ``shard='out'``: keeps a slice of the output channels
    (input replicated, output local slice or gathered); ``shard='in'``: keeps a slice of the input
    channels, consumes the local slice and all-reduces the partial sums."""
    _nd = 2

    def __init__(self, source, process_group=None, mode: str = "colwise", gather_output: bool = False, *, group=None, shard: Optional[str] = None):
        """``mode``: ``"colwise"`` (= ``shard="out"``: a slice of the output channels) or ``"rowwise"`` (= ``shard="in"``: a slice of
        the input channels, partial sums all-reduced).  ``group`` / ``shard`` are the older keyword names of the first two."""
        super().__init__()
        group = process_group if group is None else group
        shard = {"colwise": "out", "rowwise": "in"}.get(mode, mode) if shard is None else shard
        if source.groups != 1:
            raise ValueError("channel sharding supports groups == 1 only")
        if shard not in ("out", "in"):
            raise ValueError(f"mode must be 'colwise' or 'rowwise', got {mode!r}")
        self.group, self.shard, self.gather_output = group, shard, gather_output
        self.mode = "colwise" if shard == "out" else "rowwise"
        self.in_channels, self.out_channels = source.in_channels, source.out_channels
        self.kernel_size, self.stride, self.padding, self.dilation = source.kernel_size, source.stride, source.padding, source.dilation
        self.padding_mode = source.padding_mode
        if self.padding_mode != "zeros":
            raise ValueError("channel sharding supports zero padding only")
        self.step_mode = getattr(source, "step_mode", "s")
        if shard == "out":
            self.weight, self.bias = _shard_param(source.weight, 0, group), _shard_param(source.bias, 0, group)
        else:
            self.weight = _shard_param(source.weight, 1, group)
            self.bias = None if source.bias is None else nn.Parameter(source.bias.detach().clone())

    def _conv(self, x, w, b):
        f = F.conv1d if self._nd == 1 else F.conv2d
        return f(x, w, b, self.stride, self.padding, self.dilation)

    def _single(self, x):
        cdim = 1
        if self.shard == "out":
            y = self._conv(_CopyToGroup.apply(x, self.group), self.weight, self.bias)
            return _GatherFromGroup.apply(y, self.group, cdim, False) if self.gather_output else y
        if x.shape[cdim] == self.in_channels and _ws(self.group) > 1:
            x = _ScatterToGroup.apply(x, self.group, cdim)
        y = _ReduceFromGroup.apply(self._conv(x, self.weight, None), self.group)
        return y if self.bias is None else y + self.bias.view(1, -1, *([1] * self._nd))

    def forward(self, x):
        if self.step_mode == "m" and x.dim() == self._nd + 3:
            t, n = x.shape[:2]
            y = self._single(x.flatten(0, 1))
            return y.reshape(t, n, *y.shape[1:])
        return self._single(x)


class ChannelShardConv1d(_ChannelShardConv):
    _nd = 1


class ChannelShardConv2d(_ChannelShardConv):
    _nd = 2


class _ChannelShardBatchNorm(nn.Module):
    """BatchNorm over the local slice of the channels (statistics are per channel, so no communication)."""
    _cls = nn.BatchNorm2d

    def __init__(self, source, process_group=None, *, group=None):
        super().__init__()
        group = process_group if group is None else group
        self.group, self.num_features = group, source.num_features
        ws, r = _ws(group), _rank(group)
        n = _even(source.num_features, ws, "num_features")
        self.local = self._cls(n, eps=source.eps, momentum=source.momentum, affine=source.affine,
                               track_running_stats=source.track_running_stats)
        with torch.no_grad():
            for k, v in source.state_dict().items():
                getattr(self.local, k).copy_(v if v.dim() == 0 else v.narrow(0, r * n, n))
        self.local.to(next(iter(source.state_dict().values())).device if source.state_dict() else "cpu")
        self.step_mode = getattr(source, "step_mode", "s")

    def forward(self, x):
        nd = 3 if self._cls is nn.BatchNorm1d else 4
        if self.step_mode == "m" and x.dim() == nd + 1:
            t, n = x.shape[:2]
            return self.local(x.flatten(0, 1)).reshape(x.shape)
        return self.local(x)


class ChannelShardBatchNorm1d(_ChannelShardBatchNorm):
    _cls = nn.BatchNorm1d


class ChannelShardBatchNorm2d(_ChannelShardBatchNorm):
    _cls = nn.BatchNorm2d


def _shard_conv_chain(seq, group) -> int:
    """In a flat container: pair up convolutions (1st: out-sharded, 2nd: in-sharded, ...); BatchNorms
    and stateful modules between a pair work on the local channel slice.  Returns #convs sharded."""
    items = list(seq.named_children())
    conv_idx = [i for i, (_, m) in enumerate(items) if isinstance(m, (nn.Conv1d, nn.Conv2d)) and m.groups == 1]
    done = 0
    for a, b in zip(conv_idx[0::2], conv_idx[1::2]):
        first, second = items[a][1], items[b][1]
        if first.out_channels != second.in_channels or first.out_channels % _ws(group):
            continue
        between = items[a + 1:b]
        if any(not isinstance(m, (nn.modules.batchnorm._BatchNorm, base.MemoryModule, nn.MaxPool1d, nn.MaxPool2d, nn.AvgPool1d,
                                  nn.AvgPool2d, nn.Dropout, nn.Identity, layer.Dropout)) for _, m in between):
            continue
        C1 = ChannelShardConv1d if isinstance(first, nn.Conv1d) else ChannelShardConv2d
        C2 = ChannelShardConv1d if isinstance(second, nn.Conv1d) else ChannelShardConv2d
        _replace(seq, items[a][0], C1(first, group, "out"))
        _replace(seq, items[b][0], C2(second, group, "in"))
        for name, m in between:
            if isinstance(m, nn.BatchNorm1d):
                _replace(seq, name, ChannelShardBatchNorm1d(m, group))
            elif isinstance(m, nn.BatchNorm2d):
                _replace(seq, name, ChannelShardBatchNorm2d(m, group))
            elif isinstance(m, base.MemoryModule):
                cdim = 2 if getattr(m, "step_mode", "s") == "m" else 1
                _replace(seq, name, make_tensor_shard_memory_module(m, cdim, first.out_channels, group))
        done += 2
    return done


def parallelize_snn_conv_blocks(module: nn.Module, device_mesh, roots: Sequence[str], tp_mesh_dim: int = 0) -> nn.Module:
    """Channel-shard the convolution chains found in the flat containers under ``roots``."""
    group = _group_of(device_mesh, tp_mesh_dim)
    named = dict(module.named_modules())
    for root in roots:
        if root not in named:
            raise KeyError(f"Unknown conv tensor-parallel root '{root}'.")
        for sub in [m for m in named[root].modules() if isinstance(m, (nn.Sequential, nn.ModuleList))]:
            _shard_conv_chain(sub, group)
    return module


# ------------------------------------------------------------------------------------ Spikformer
def _shard_heads_qkv(attn, group) -> None:
    """q, k and v projections (one fused 1x1 convolution with 3 * dim outputs, followed by BatchNorm)
    keep the heads of this rank; the output projection consumes them and all-reduces."""
    ws, r = _ws(group), _rank(group)
    dim, heads = attn.dim, attn.num_heads
    local_heads = _even(heads, ws, "num_heads")
    hd = dim // heads
    conv, bn = attn.qkv_conv_bn[0], attn.qkv_conv_bn[1]
    rows = torch.cat([torch.arange(part * dim + r * local_heads * hd, part * dim + (r + 1) * local_heads * hd) for part in range(3)])
    new_conv = nn.Conv1d(dim, rows.numel(), 1, bias=conv.bias is not None).to(conv.weight.device, conv.weight.dtype)
    new_bn = nn.BatchNorm1d(rows.numel(), eps=bn.eps, momentum=bn.momentum).to(conv.weight.device)
    with torch.no_grad():
        rows = rows.to(conv.weight.device)
        new_conv.weight.copy_(conv.weight[rows])
        if conv.bias is not None:
            new_conv.bias.copy_(conv.bias[rows])
        for k in ("weight", "bias", "running_mean", "running_var"):
            getattr(new_bn, k).copy_(getattr(bn, k)[rows])
        new_bn.num_batches_tracked.copy_(bn.num_batches_tracked)
    attn.qkv_conv_bn[0] = _CopyInput(new_conv, group)
    attn.qkv_conv_bn[1] = new_bn
    attn.num_heads = local_heads
    proj = attn.proj_conv_bn[0]
    attn.proj_conv_bn[0] = ChannelShardConv1d(proj, group, "in")


class _CopyInput(nn.Module):
    """Marks the point where a replicated activation enters sharded compute (gradient all-reduce)."""

    def __init__(self, inner: nn.Module, group):
        super().__init__()
        self.inner, self.group = inner, group

    def forward(self, x):
        return self.inner(_CopyToGroup.apply(x, self.group))


def parallelize_spikformer_blocks(module: nn.Module, device_mesh, roots: Sequence[str] = ("blocks",), tp_mesh_dim: int = 0) -> nn.Module:
    """Shard every Spikformer block under ``roots``: attention heads across ranks (q/k/v column-
    parallel, projection row-parallel) and the MLP hidden channels (fc1 column-, fc2 row-parallel).
    The block output equals the unsharded block's output."""
    group = _group_of(device_mesh, tp_mesh_dim)
    named = dict(module.named_modules())
    for root in roots:
        if root not in named:
            raise KeyError(f"Unknown Spikformer tensor-parallel root '{root}'.")
        for blk in [m for m in named[root].modules() if hasattr(m, "attn") and hasattr(m, "mlp")]:
            _shard_heads_qkv(blk.attn, group)
            mlp = blk.mlp
            fc1, bn1 = mlp.fc1[0], mlp.fc1[1]
            mlp.fc1[0] = ChannelShardConv1d(fc1, group, "out")
            mlp.fc1[1] = ChannelShardBatchNorm1d(bn1, group).local
            mlp.fc2[0] = ChannelShardConv1d(mlp.fc2[0], group, "in")
            if hasattr(blk, "fused") or hasattr(module, "fused"):
                pass
    if hasattr(module, "fused"):
        module.fused = False          # the fused single-GPU schedule assumes unsharded blocks
    return module


def parallelize_spikformer_patch_stem(module: nn.Module, device_mesh, roots: Sequence[str] = ("patch_embed",),
                                      tp_mesh_dim: int = 0) -> nn.Module:
    """Channel-shard the convolution stages of the patch stem pairwise (stage 2k out-sharded, stage
    2k+1 in-sharded)."""
    group = _group_of(device_mesh, tp_mesh_dim)
    named = dict(module.named_modules())
    for root in roots:
        if root not in named:
            raise KeyError(f"Unknown patch-stem tensor-parallel root '{root}'.")
        stem = named[root]
        stages = list(getattr(stem, "stages", []))
        for a, b in zip(stages[0::2], stages[1::2]):
            ca, cb = a.conv_bn.block[0], b.conv_bn.block[0]
            if ca.out_channels != cb.in_channels or ca.out_channels % _ws(group):
                continue
            a.conv_bn.block[0] = ChannelShardConv2d(ca, group, "out")
            a.conv_bn.block[1] = ChannelShardBatchNorm2d(a.conv_bn.block[1], group).local
            b.conv_bn.block[0] = ChannelShardConv2d(cb, group, "in")
    if hasattr(module, "fused"):
        module.fused = False
    return module


def __getattr__(name: str):
    # type tuples the VGG channel-sharding plan matches against, under the reference's names
    if name in ("Conv2dLike", "BatchNorm2dLike"):
        from ..activation_based import layer
        return (nn.Conv2d, layer.Conv2d) if name == "Conv2dLike" else (nn.BatchNorm2d, layer.BatchNorm2d)
    raise AttributeError(name)
