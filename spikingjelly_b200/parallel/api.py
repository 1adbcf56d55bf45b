"""Analyze -> Plan -> Apply, the three-call front end of distributed training
(``spikingjelly/activation_based/distributed/api.py:39-310``):

    analysis = analyze(model)                                   # what is stateful, what can be sharded
    decision = plan(analysis=analysis, objective="memory", topology={"dp": 4, "tp": 2}, backend="cuda", batch_size=64)
    runtime  = apply(model=model, plan=decision)                # configured model + mesh + helpers

``plan`` starts from the recommender's answer for the objective, lets an explicit ``mode`` override it, then fits the
result to the topology and to what the analysis found.  Each adjustment is a small function that either returns a note
or raises; the notes end up in ``SNNDistributedPlan.notes``."""
from __future__ import annotations

from typing import List, Mapping, Optional, Sequence, Union

import torch.nn as nn

from ..logger import logger
from . import _schema
from .adapters import build_distributed_runtime, resolve_adapter
from .analysis import SNNDistributedAnalysis, analyze_snn_distributed_capability
from .data_parallel import unwrap_parallel_module
from .planner import (SNN_DISTRIBUTED_PREFERENCES, DistributedFeatureSet, SNNDistributedPlan, TensorParallelStyle,
                      recommend_snn_distributed_strategy)
from .runtime import SNNDistributedRuntime
from .topology import SNNDistributedTopology

__all__ = ["analyze", "plan", "apply"]

_MODES = ("none", "dp", "tp", "fsdp2", "fsdp2_tp", "pp")
_TENSOR_PARALLEL_MODES = ("tp", "fsdp2_tp")


def _no_pipeline_here():
    raise NotImplementedError("mode 'pp': pipeline parallelism needs an example input to cut the model into stages and to cost "
                              "them, which analyze/plan/apply does not have; use the pipeline builders in parallel.pipeline")


def _as_topology(topology) -> SNNDistributedTopology:
    return topology if isinstance(topology, SNNDistributedTopology) else SNNDistributedTopology.from_mapping(topology)


def analyze(model: nn.Module, *, roots: Optional[Sequence[str]] = None) -> SNNDistributedAnalysis:
    """Scan ``model`` (or only what lies under ``roots``) for stateful modules and tensor-parallel candidates."""
    found = analyze_snn_distributed_capability(model, tensor_parallel_roots=roots)
    logger.info("analysis: %d stateful, %d shardable, %d convolution(s) left whole (roots=%s)", len(found.memory_module_names),
                len(found.tensor_parallel_candidate_names), len(found.unsupported_tensor_parallel_names), roots)
    return found


def _fit_mode_to_topology(wanted: str, forced: bool, topo: SNNDistributedTopology, notes: List[str]) -> str:
    if wanted != "fsdp2_tp" or topo.has("dp", "tp"):
        return wanted
    if forced:
        raise ValueError(f"mode 'fsdp2_tp' requires both 'dp' and 'tp' axes in the topology, which has {topo.ordered_dim_names}")
    fitted = "tp" if topo.has("tp") else "fsdp2"
    notes.append(f"the recommended 'fsdp2_tp' needs a 'dp' and a 'tp' axis; with axes {topo.ordered_dim_names} it was reduced to '{fitted}'")
    return fitted


def _check_tensor_parallel(mode: str, analysis: SNNDistributedAnalysis, explicit: Optional[Mapping[str, TensorParallelStyle]]) -> None:
    sharded = mode in _TENSOR_PARALLEL_MODES
    if sharded and not analysis.tensor_parallel_candidate_names:
        raise ValueError(f"mode '{mode}' requires at least one tensor-parallel candidate and the analysis found none")
    if explicit is None:
        return
    if not sharded:
        raise ValueError(f"tensor_parallel_plan was given but mode '{mode}' does no tensor parallelism (use 'tp' or 'fsdp2_tp')")
    if len(explicit) == 0:
        raise ValueError("tensor_parallel_plan is empty; pass None to have the plan built automatically")
    strangers = sorted(set(explicit) - set(analysis.tensor_parallel_candidate_names))
    if strangers:
        raise ValueError(f"tensor_parallel_plan names modules outside the analysis candidates: {strangers}")


def _optimizer_strategy(mode: str, recommended: str, features: DistributedFeatureSet, notes: List[str]) -> str:
    if mode != "dp":
        return "none"                    # optimizer-state sharding is offered for pure data parallelism only
    if recommended == "zero" and not features.allow_zero_optimizer:
        notes.append("ZeRO optimizer sharding was switched off by the feature set; every rank keeps the full optimizer state")
        return "none"
    return recommended


def plan(*, analysis: SNNDistributedAnalysis, objective: str, topology: Union[Mapping[str, int], SNNDistributedTopology], backend: str,
         batch_size: int, model_family: Optional[str] = None, mode: Optional[str] = None,
         features: Optional[DistributedFeatureSet] = None,
         tensor_parallel_plan: Optional[Mapping[str, TensorParallelStyle]] = None) -> SNNDistributedPlan:
    """Decide mode, optimizer sharding and memopt level for ``objective`` (``speed | memory | capacity``) on ``topology``."""
    objective = _schema.one_of(objective, SNN_DISTRIBUTED_PREFERENCES, "objective")
    forced = None if mode is None else _schema.one_of(mode, _MODES, "mode")
    if forced == "pp":
        _no_pipeline_here()
    topo = _as_topology(topology)
    features = DistributedFeatureSet() if features is None else features
    family = model_family or "generic"
    advice = recommend_snn_distributed_strategy(model=family, world_size=topo.world_size, prefer=objective, batch_size=batch_size,
                                                backend=backend, pipelining_available=False)
    notes = list(analysis.notes)
    chosen = _fit_mode_to_topology(forced or advice.mode, forced is not None, topo, notes)
    _check_tensor_parallel(chosen, analysis, tensor_parallel_plan)
    decision = SNNDistributedPlan(
        mode=chosen, objective=objective, topology=topo, model_family=family, backend=backend, batch_size=batch_size,
        optimizer_strategy=_optimizer_strategy(chosen, advice.optimizer_sharding, features, notes), memopt_level=advice.memopt_level,
        rationale=tuple(advice.rationale), notes=tuple(notes), tensor_parallel_roots=analysis.tensor_parallel_roots,
        tensor_parallel_plan=tensor_parallel_plan, experimental_features=features)
    logger.info("plan: mode=%s for objective=%s on mesh %s (optimizer=%s, memopt level %d, explicit TP plan: %s)", decision.mode,
                objective, topo.mesh_shape, decision.optimizer_strategy, decision.memopt_level, tensor_parallel_plan is not None)
    return decision


def apply(*, model: nn.Module, plan: SNNDistributedPlan, device_type: str = "cuda", device_mesh=None) -> SNNDistributedRuntime:
    """Carry out ``plan`` on ``model``; known model families go through their adapter (which knows what to shard)."""
    if plan.mode == "pp":
        _no_pipeline_here()
    model = unwrap_parallel_module(model)
    topo = _as_topology(plan.topology)
    if device_mesh is not None:
        ranks = int(device_mesh.mesh.numel())
        if ranks != topo.world_size:
            raise ValueError(f"device_mesh has {ranks} rank(s) but the plan was made for {topo.world_size}")
    opted_in = plan.experimental_features.allow_experimental_conv_tp or plan.experimental_features.allow_experimental_spikformer_tp
    adapter = resolve_adapter(model, plan.model_family) if (plan.mode in ("tp", "fsdp2", "fsdp2_tp") or opted_in) else None
    if adapter is None:
        return build_distributed_runtime(model, plan, device_type=device_type, device_mesh=device_mesh,
                                         tensor_parallel_roots=plan.tensor_parallel_roots)
    return adapter.apply(model, plan, device_type=device_type, device_mesh=device_mesh)
