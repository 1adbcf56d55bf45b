"""Analyze -> Plan -> Apply: the three-call front end of distributed SNN training.
Parity: ``spikingjelly/activation_based/distributed/api.py:24-310``."""
from __future__ import annotations

from typing import Mapping, Optional, Sequence, Union

import torch.nn as nn

from ..logger import logger
from .adapters import build_distributed_runtime, resolve_adapter
from .analysis import SNNDistributedAnalysis, analyze_snn_distributed_capability
from .data_parallel import unwrap_parallel_module
from .planner import (SNN_DISTRIBUTED_PREFERENCES, DistributedFeatureSet, SNNDistributedPlan, TensorParallelStyle,
                      recommend_snn_distributed_strategy)
from .runtime import SNNDistributedRuntime
from .topology import SNNDistributedTopology

__all__ = ["analyze", "plan", "apply"]

_PP_MESSAGE = ("Pipeline parallelism ('pp') is not supported by the unified analyze/plan/apply API because it needs an example "
               "input to cut the model and cost the stages. Please use the dedicated pipeline configuration path directly.")


def _normalize_mode(mode: Optional[str]) -> Optional[str]:
    if mode is None:
        return None
    mode = mode.lower()
    valid = ("none", "dp", "tp", "fsdp2", "fsdp2_tp", "pp")
    if mode not in valid:
        raise ValueError(f"Unsupported mode='{mode}'. Expected one of {valid}.")
    if mode == "pp":
        raise NotImplementedError(_PP_MESSAGE)
    return mode


def analyze(model: nn.Module, *, roots: Optional[Sequence[str]] = None) -> SNNDistributedAnalysis:
    """Find stateful modules and tensor-parallel candidates (optionally only under ``roots``)."""
    a = analyze_snn_distributed_capability(model, tensor_parallel_roots=roots)
    logger.info("distributed_analysis_summary memory_modules=%s tensor_parallel_candidates=%s unsupported_tensor_parallel=%s roots=%s",
                len(a.memory_module_names), len(a.tensor_parallel_candidate_names), len(a.unsupported_tensor_parallel_names), roots)
    return a


def plan(*, analysis: SNNDistributedAnalysis, objective: str, topology: Union[Mapping[str, int], SNNDistributedTopology], backend: str,
         batch_size: int, model_family: Optional[str] = None, mode: Optional[str] = None,
         features: Optional[DistributedFeatureSet] = None,
         tensor_parallel_plan: Optional[Mapping[str, TensorParallelStyle]] = None) -> SNNDistributedPlan:
    """Choose mode, optimizer sharding and memopt level for ``objective`` in (speed, memory, capacity) on
    ``topology`` (``{"dp": 4, "tp": 2}``); ``mode`` overrides the recommendation."""
    objective = objective.lower()
    if objective not in SNN_DISTRIBUTED_PREFERENCES:
        raise ValueError(f"Unsupported objective='{objective}'. Expected one of {SNN_DISTRIBUTED_PREFERENCES}.")
    topo = topology if isinstance(topology, SNNDistributedTopology) else SNNDistributedTopology.from_mapping(topology)
    features = features or DistributedFeatureSet()
    family = model_family or "generic"
    dims = topo.ordered_dim_names
    rec = recommend_snn_distributed_strategy(model=family, world_size=topo.world_size, prefer=objective, batch_size=batch_size,
                                             backend=backend, pipelining_available=False)
    mode = _normalize_mode(mode)
    notes = list(analysis.notes)
    selected = mode or rec.mode
    if selected == "fsdp2_tp" and not {"dp", "tp"} <= set(dims):
        if mode is not None:
            raise ValueError("Hybrid 'fsdp2_tp' mode requires both 'dp' and 'tp' dimensions in the topology.")
        selected = "tp" if "tp" in dims else "fsdp2"
        notes.append(f"Recommended 'fsdp2_tp' was reduced to '{selected}' for topology dimensions {dims}.")
    if selected in ("tp", "fsdp2_tp") and not analysis.tensor_parallel_candidate_names:
        raise ValueError(f"mode='{selected}' requires at least one tensor-parallel candidate, but analysis found none.")
    if tensor_parallel_plan is not None:
        if selected not in ("tp", "fsdp2_tp"):
            raise ValueError("tensor_parallel_plan requires mode='tp' or mode='fsdp2_tp'.")
        if not tensor_parallel_plan:
            raise ValueError("tensor_parallel_plan must not be empty.")
        unknown = set(tensor_parallel_plan) - set(analysis.tensor_parallel_candidate_names)
        if unknown:
            raise ValueError(f"tensor_parallel_plan contains modules outside the analysis candidates: {sorted(unknown)!r}.")
    optimizer_strategy = rec.optimizer_sharding
    if selected != "dp" or not features.allow_zero_optimizer:
        optimizer_strategy = "none"
        if selected == "dp" and not features.allow_zero_optimizer:
            notes.append("Zero optimizer was disabled by DistributedFeatureSet; planner fell back to optimizer_strategy='none'.")
    p = SNNDistributedPlan(mode=selected, objective=objective, topology=topo, model_family=family, backend=backend, batch_size=batch_size,
                           optimizer_strategy=optimizer_strategy, memopt_level=rec.memopt_level, rationale=tuple(rec.rationale),
                           notes=tuple(notes), tensor_parallel_roots=analysis.tensor_parallel_roots,
                           tensor_parallel_plan=tensor_parallel_plan, experimental_features=features)
    logger.info("distributed_plan_summary mode=%s objective=%s backend=%s world_size=%s mesh_shape=%s optimizer_strategy=%s "
                "memopt_level=%s tensor_parallel_plan=%s", p.mode, p.objective, p.backend, topo.world_size, topo.mesh_shape,
                p.optimizer_strategy, p.memopt_level, p.tensor_parallel_plan is not None)
    return p


def apply(*, model: nn.Module, plan: SNNDistributedPlan, device_type: str = "cuda", device_mesh=None) -> SNNDistributedRuntime:
    """Configure ``model`` according to ``plan`` (through the model family's adapter where one exists)."""
    model = unwrap_parallel_module(model)
    topo = plan.topology if isinstance(plan.topology, SNNDistributedTopology) else SNNDistributedTopology.from_mapping(plan.topology)
    if device_mesh is not None and int(device_mesh.mesh.numel()) != topo.world_size:
        raise ValueError(f"device_mesh spans {int(device_mesh.mesh.numel())} ranks, but plan.topology.world_size={topo.world_size}.")
    if plan.mode == "pp":
        raise NotImplementedError(_PP_MESSAGE)
    use_adapter = plan.mode in ("tp", "fsdp2", "fsdp2_tp") or plan.experimental_features.allow_experimental_conv_tp \
        or plan.experimental_features.allow_experimental_spikformer_tp
    adapter = resolve_adapter(model, plan.model_family) if use_adapter else None
    if adapter is not None:
        return adapter.apply(model, plan, device_type=device_type, device_mesh=device_mesh)
    return build_distributed_runtime(model, plan, device_type=device_type, device_mesh=device_mesh,
                                     tensor_parallel_roots=plan.tensor_parallel_roots)
