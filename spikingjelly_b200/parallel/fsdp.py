"""FSDP2 (``torch.distributed.fsdp.fully_shard``) over chosen sub-trees of an SNN
(``spikingjelly/activation_based/distributed/fsdp.py:13-105``).  Parameter sharding is not a path this package owns
kernels for: torch's implementation over NCCL is used as it is, this module only decides what gets wrapped."""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn

from .mesh import MeshView

try:
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
except ImportError:                                       # pragma: no cover
    MixedPrecisionPolicy = fully_shard = None
FSDP2_AVAILABLE = fully_shard is not None

__all__ = ["FSDP2_AVAILABLE", "fully_shard_snn_module", "apply_snn_fsdp2"]


def _build_fsdp_mp_policy(param_dtype, reduce_dtype, output_dtype):
    """A ``MixedPrecisionPolicy`` when any dtype is given, else ``None`` (FSDP2's default)."""
    asked = any(d is not None for d in (param_dtype, reduce_dtype, output_dtype))
    if not asked or MixedPrecisionPolicy is None:
        return None
    return MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype, output_dtype=output_dtype)


def fully_shard_snn_module(module: nn.Module, device_mesh, shard_roots: Optional[Sequence[str]] = None,
                           shard_module_root: bool = True, root_reshard_after_forward: Optional[bool] = False, mp_policy=None) -> nn.Module:
    """Wrap each path of ``shard_roots`` as its own FSDP unit, then the model itself unless ``shard_module_root`` is false
    (``""`` among the roots also asks for the model).  The outermost unit keeps its parameters gathered after forward by
    default, because an SNN's backward starts at once and would only gather them again."""
    if not FSDP2_AVAILABLE:
        raise RuntimeError("this PyTorch build has no torch.distributed.fsdp.fully_shard")
    by_path = dict(module.named_modules())
    wanted = list(shard_roots or ())
    missing = [p for p in wanted if p not in by_path]
    if missing:
        raise KeyError(f"fsdp shard roots not found in the model: {missing}")
    options = {} if mp_policy is None else {"mp_policy": mp_policy}
    for path in wanted:
        if path:
            fully_shard(by_path[path], mesh=device_mesh, **options)
    if shard_module_root or "" in wanted:
        fully_shard(module, mesh=device_mesh, reshard_after_forward=root_reshard_after_forward, **options)
    return module


def apply_snn_fsdp2(module: nn.Module, device_mesh, dp_mesh_dim: Optional[int] = None, shard_roots: Optional[Sequence[str]] = None,
                    shard_module_root: bool = True, root_reshard_after_forward: Optional[bool] = False,
                    param_dtype: Optional[torch.dtype] = None, reduce_dtype: Optional[torch.dtype] = None,
                    output_dtype: Optional[torch.dtype] = None) -> nn.Module:
    """:func:`fully_shard_snn_module` over the data-parallel axis of ``device_mesh`` (axis 0 unless told otherwise)."""
    axis_mesh = MeshView(device_mesh).axis_submesh(0 if dp_mesh_dim is None else dp_mesh_dim)
    policy = _build_fsdp_mp_policy(param_dtype, reduce_dtype, output_dtype)
    return fully_shard_snn_module(module, axis_mesh, shard_roots, shard_module_root, root_reshard_after_forward, policy)
