"""``configure_snn_distributed(module, config)``: build the mesh and apply tensor parallelism,
FSDP2 and data parallelism in that order.  Parity: ``spikingjelly/activation_based/distributed/execution.py:46-230``."""
from __future__ import annotations

import warnings
from typing import Optional, Tuple

import torch
import torch.nn as nn

from ..logger import logger
from .analysis import SNNDistributedAnalysis, analyze_snn_distributed_capability
from .config import SNNDistributedConfig
from .data_parallel import prepare_snn_data_parallel
from .fsdp import _build_fsdp_mp_policy, fully_shard_snn_module
from .mesh import _resolve_dp_group_from_mesh, _resolve_mesh_dim_group, _resolve_mesh_submesh, build_device_mesh
from .tensor_parallel import (auto_build_tensor_parallel_plan, parallelize_snn_conv_blocks, parallelize_snn_module,
                              parallelize_spikformer_blocks, parallelize_spikformer_patch_stem, wrap_tp_memory_modules)

__all__ = ["configure_snn_distributed"]


def _validate_mesh_dims(config: SNNDistributedConfig, ndim: int) -> None:
    tp = config.mode in ("tp", "fsdp2_tp")
    if config.mode in ("dp", "fsdp2", "fsdp2_tp") and ndim > 1 and config.dp_mesh_dim is None:
        raise ValueError(f"dp_mesh_dim must be specified for mode={config.mode!r} on a multi-dimensional DeviceMesh.")
    for name, dim in (("tp_mesh_dim", config.tp_mesh_dim), ("dp_mesh_dim", config.dp_mesh_dim)):
        if dim is not None and not 0 <= dim < ndim:
            raise ValueError(f"{name}={dim} is out of range for a mesh with {ndim} dimensions.")
    if tp and config.dp_mesh_dim == config.tp_mesh_dim:
        raise ValueError(f"tp_mesh_dim and dp_mesh_dim must be different when tensor parallelism is enabled, but both are {config.tp_mesh_dim}.")


def configure_snn_distributed(module: nn.Module, config: SNNDistributedConfig) -> Tuple[nn.Module, Optional[object], SNNDistributedAnalysis]:
    """Returns ``(configured module, device mesh or None, analysis)``."""
    tp = config.mode in ("tp", "fsdp2_tp")
    analysis = analyze_snn_distributed_capability(module, tensor_parallel_roots=config.tensor_parallel_roots)
    if config.device_mesh is None and config.mode == "none":
        logger.info("distributed_configuration_summary mode=%s device_type=%s mesh_shape=None tensor_parallel=%s fsdp2=False "
                    "data_parallel=False memory_modules=%s tensor_parallel_candidates=%s", config.mode, config.device_type, tp,
                    len(analysis.memory_module_names), len(analysis.tensor_parallel_candidate_names))
        return module, None, analysis

    if config.device_mesh is None:
        ndim = len(config.mesh_shape) if config.mesh_shape is not None else 1
        _validate_mesh_dims(config, ndim)
        names = None
        if ndim > 1:
            names = [f"mesh_dim_{i}" for i in range(ndim)]
            names[config.tp_mesh_dim] = "tp"
            if config.dp_mesh_dim is not None:
                names[config.dp_mesh_dim] = "dp"
            names = tuple(names)
        mesh = build_device_mesh(config.device_type, config.mesh_shape, names)
    else:
        if config.mesh_shape is not None:
            warnings.warn("`device_mesh` was supplied explicitly; `mesh_shape` is ignored.", UserWarning, stacklevel=2)
        mesh = config.device_mesh
        _validate_mesh_dims(config, int(mesh.mesh.ndim))

    if tp and config.conv_tensor_parallel_roots:
        module = parallelize_snn_conv_blocks(module, mesh, config.conv_tensor_parallel_roots, config.tp_mesh_dim)
    if tp and config.spikformer_tensor_parallel_roots:
        module = parallelize_spikformer_blocks(module, mesh, config.spikformer_tensor_parallel_roots, config.tp_mesh_dim)
    if tp and config.spikformer_patch_stem_tensor_parallel_roots:
        module = parallelize_spikformer_patch_stem(module, mesh, config.spikformer_patch_stem_tensor_parallel_roots, config.tp_mesh_dim)
    if tp and (config.tensor_parallel_plan is not None or config.auto_tensor_parallel):
        plan = dict(config.tensor_parallel_plan) if config.tensor_parallel_plan is not None else \
            auto_build_tensor_parallel_plan(module, tensor_parallel_roots=config.tensor_parallel_roots)
        group = _resolve_mesh_dim_group(mesh, config.tp_mesh_dim)
        module = wrap_tp_memory_modules(module, plan, group)
        module = parallelize_snn_module(module, mesh, plan, config.tp_mesh_dim)

    if config.mode in ("fsdp2", "fsdp2_tp"):
        fsdp_mesh = _resolve_mesh_submesh(mesh, config.dp_mesh_dim if config.dp_mesh_dim is not None else 0)
        module = fully_shard_snn_module(module, fsdp_mesh, config.fsdp_shard_roots, config.fsdp_shard_module_root,
                                        config.fsdp_root_reshard_after_forward,
                                        _build_fsdp_mp_policy(config.fsdp_param_dtype, config.fsdp_reduce_dtype, config.fsdp_output_dtype))
    if config.mode == "dp":
        ids = [torch.cuda.current_device()] if config.device_type == "cuda" and torch.cuda.is_available() else None
        module = prepare_snn_data_parallel(module, process_group=_resolve_dp_group_from_mesh(mesh, config.dp_mesh_dim), device_ids=ids,
                                           broadcast_buffers=config.broadcast_buffers,
                                           find_unused_parameters=config.find_unused_parameters, static_graph=config.static_graph)
    logger.info("distributed_configuration_summary mode=%s device_type=%s mesh_shape=%s tensor_parallel=%s fsdp2=%s data_parallel=%s "
                "memory_modules=%s tensor_parallel_candidates=%s", config.mode, config.device_type,
                tuple(int(v) for v in mesh.mesh.shape), tp, config.mode in ("fsdp2", "fsdp2_tp"), config.mode == "dp",
                len(analysis.memory_module_names), len(analysis.tensor_parallel_candidate_names))
    return module, mesh, analysis
