"""FSDP2 (``torch.distributed.fsdp.fully_shard``) applied to chosen roots of an SNN.  Parameter
sharding is not on a hot path the package owns kernels for, so torch's implementation over NCCL is
used as is.  Parity: ``spikingjelly/activation_based/distributed/fsdp.py:13-105``."""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn

from .mesh import _resolve_mesh_submesh

try:
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    FSDP2_AVAILABLE = True
except ImportError:                                       # pragma: no cover
    MixedPrecisionPolicy = None
    fully_shard = None
    FSDP2_AVAILABLE = False

__all__ = ["FSDP2_AVAILABLE", "fully_shard_snn_module", "apply_snn_fsdp2"]


def _build_fsdp_mp_policy(param_dtype, reduce_dtype, output_dtype):
    if MixedPrecisionPolicy is None or (param_dtype is None and reduce_dtype is None and output_dtype is None):
        return None
    return MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype, output_dtype=output_dtype)


def fully_shard_snn_module(module: nn.Module, device_mesh, shard_roots: Optional[Sequence[str]] = None,
                           shard_module_root: bool = True, root_reshard_after_forward: Optional[bool] = False, mp_policy=None) -> nn.Module:
    """``fully_shard`` every module path in ``shard_roots`` (``""`` = the model itself), then the model
    (unless ``shard_module_root`` is false).  The root keeps its parameters gathered after forward by
    default: an SNN's backward starts right away."""
    if not FSDP2_AVAILABLE:
        raise RuntimeError("FSDP2 fully_shard is unavailable in the current PyTorch build.")
    named = dict(module.named_modules())
    extra = {} if mp_policy is None else {"mp_policy": mp_policy}
    root_listed = False
    for name in list(shard_roots or []):
        if name not in named:
            raise KeyError(f"Unknown FSDP shard root '{name}'.")
        if name == "":
            root_listed = True
            continue
        fully_shard(named[name], mesh=device_mesh, **extra)
    if shard_module_root or root_listed:
        fully_shard(module, mesh=device_mesh, reshard_after_forward=root_reshard_after_forward, **extra)
    return module


def apply_snn_fsdp2(module: nn.Module, device_mesh, dp_mesh_dim: Optional[int] = None, shard_roots: Optional[Sequence[str]] = None,
                    shard_module_root: bool = True, root_reshard_after_forward: Optional[bool] = False,
                    param_dtype: Optional[torch.dtype] = None, reduce_dtype: Optional[torch.dtype] = None,
                    output_dtype: Optional[torch.dtype] = None) -> nn.Module:
    mesh = _resolve_mesh_submesh(device_mesh, dp_mesh_dim if dp_mesh_dim is not None else 0)
    return fully_shard_snn_module(module, mesh, shard_roots, shard_module_root, root_reshard_after_forward,
                                  _build_fsdp_mp_policy(param_dtype, reduce_dtype, output_dtype))
