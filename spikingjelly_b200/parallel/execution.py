"""``configure_snn_distributed(module, config)``: carry out one :class:`SNNDistributedConfig`
(``spikingjelly/activation_based/distributed/execution.py:72-230``).

The work is a fixed sequence of passes over the model — channel-sharded convolution stacks, Spikformer blocks and patch
stem, linear tensor parallelism, FSDP2, data parallelism — each of which looks at the configuration, decides whether it has
anything to do and returns the (possibly wrapped) model.  The mesh comes first: the caller's, or a new one named after the
configuration's axes."""
from __future__ import annotations

import warnings
from typing import Callable, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..logger import logger
from .analysis import SNNDistributedAnalysis, analyze_snn_distributed_capability
from .config import SNNDistributedConfig
from .data_parallel import prepare_snn_data_parallel
from .fsdp import _build_fsdp_mp_policy, fully_shard_snn_module
from .mesh import MeshView, build_device_mesh
from .tensor_parallel import (auto_build_tensor_parallel_plan, parallelize_snn_conv_blocks, parallelize_snn_module,
                              parallelize_spikformer_blocks, parallelize_spikformer_patch_stem, wrap_tp_memory_modules)

__all__ = ["configure_snn_distributed"]

_Pass = Callable[[nn.Module, SNNDistributedConfig, object], nn.Module]


def _obtain_mesh(config: SNNDistributedConfig):
    if config.device_mesh is not None:
        if config.mesh_shape is not None:
            warnings.warn("both device_mesh and mesh_shape were given; the existing mesh is used and mesh_shape ignored", UserWarning,
                          stacklevel=3)
        config.check_axes(int(config.device_mesh.mesh.ndim))
        return config.device_mesh
    ndim = 1 if config.mesh_shape is None else len(config.mesh_shape)
    config.check_axes(ndim)
    return build_device_mesh(config.device_type, config.mesh_shape, config.axis_names(ndim))


def _channel_sharding(module, config, mesh):
    if not config.uses_tensor_parallel:
        return module
    for roots, shard in ((config.conv_tensor_parallel_roots, parallelize_snn_conv_blocks),
                         (config.spikformer_tensor_parallel_roots, parallelize_spikformer_blocks),
                         (config.spikformer_patch_stem_tensor_parallel_roots, parallelize_spikformer_patch_stem)):
        if roots:
            module = shard(module, mesh, roots, config.tp_mesh_dim)
    return module


def _linear_tensor_parallel(module, config, mesh):
    explicit = config.tensor_parallel_plan
    if not config.uses_tensor_parallel or (explicit is None and not config.auto_tensor_parallel):
        return module
    styles = dict(explicit) if explicit is not None else auto_build_tensor_parallel_plan(module, tensor_parallel_roots=config.tensor_parallel_roots)
    module = wrap_tp_memory_modules(module, styles, MeshView(mesh).axis_group(config.tp_mesh_dim))
    return parallelize_snn_module(module, mesh, styles, config.tp_mesh_dim)


def _parameter_sharding(module, config, mesh):
    if not config.uses_fsdp:
        return module
    axis_mesh = MeshView(mesh).axis_submesh(0 if config.dp_mesh_dim is None else config.dp_mesh_dim)
    policy = _build_fsdp_mp_policy(config.fsdp_param_dtype, config.fsdp_reduce_dtype, config.fsdp_output_dtype)
    return fully_shard_snn_module(module, axis_mesh, config.fsdp_shard_roots, config.fsdp_shard_module_root,
                                  config.fsdp_root_reshard_after_forward, policy)


def _data_parallel(module, config, mesh):
    if not config.uses_data_parallel:
        return module
    on_gpu = config.device_type == "cuda" and torch.cuda.is_available()
    group = None if config.dp_mesh_dim is None else MeshView(mesh).axis_group(config.dp_mesh_dim)
    return prepare_snn_data_parallel(module, process_group=group, device_ids=[torch.cuda.current_device()] if on_gpu else None,
                                     broadcast_buffers=config.broadcast_buffers, find_unused_parameters=config.find_unused_parameters,
                                     static_graph=config.static_graph)


#: order matters: shard inside the model first, wrap the whole of it last
_PASSES: Sequence[_Pass] = (_channel_sharding, _linear_tensor_parallel, _parameter_sharding, _data_parallel)


def configure_snn_distributed(module: nn.Module, config: SNNDistributedConfig) -> Tuple[nn.Module, Optional[object], SNNDistributedAnalysis]:
    """Returns ``(configured module, device mesh or None, analysis)``.  Mode ``none`` without a mesh changes nothing."""
    analysis = analyze_snn_distributed_capability(module, tensor_parallel_roots=config.tensor_parallel_roots)
    if config.mode == "none" and config.device_mesh is None:
        logger.info("distributed set-up: mode none, model left as it is (%d stateful module(s))", len(analysis.memory_module_names))
        return module, None, analysis
    mesh = _obtain_mesh(config)
    for run in _PASSES:
        module = run(module, config, mesh)
    logger.info("distributed set-up: mode %s on a %s mesh (%d stateful module(s), %d tensor-parallel candidate(s))", config.mode,
                tuple(int(s) for s in mesh.mesh.shape), len(analysis.memory_module_names), len(analysis.tensor_parallel_candidate_names))
    return module, mesh, analysis
