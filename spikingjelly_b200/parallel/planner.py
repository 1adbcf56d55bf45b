"""Strategy recommendation and the immutable execution plan of Analyze -> Plan -> Apply.
Parity: ``spikingjelly/activation_based/distributed/planner.py:56-490``."""
from __future__ import annotations

from dataclasses import dataclass, replace
from types import MappingProxyType
from typing import Any, List, Mapping, Optional, Tuple, Union

from .topology import SNNDistributedTopology

__all__ = ["SNN_DISTRIBUTED_PREFERENCES", "DistributedFeatureSet", "SNNDistributedPlan", "SNNDistributedRecommendation",
           "TensorParallelStyle", "recommended_pipeline_microbatches", "recommend_snn_distributed_strategy",
           "FSDP2_AVAILABLE", "ZERO_REDUNDANCY_OPTIMIZER_AVAILABLE", "PIPELINING_AVAILABLE", "TENSOR_PARALLEL_AVAILABLE"]

TensorParallelStyle = Union[str, Any]
SNN_DISTRIBUTED_PREFERENCES = ("speed", "memory", "capacity")


def _has(path: str, name: str) -> bool:
    try:
        return hasattr(__import__(path, fromlist=[name]), name)
    except ImportError:
        return False


FSDP2_AVAILABLE = _has("torch.distributed.fsdp", "fully_shard")
ZERO_REDUNDANCY_OPTIMIZER_AVAILABLE = _has("torch.distributed.optim", "ZeroRedundancyOptimizer")
PIPELINING_AVAILABLE = _has("torch.distributed.pipelining", "PipelineStage")
TENSOR_PARALLEL_AVAILABLE = True          # tensor parallelism is implemented on plain process groups in this package


@dataclass(frozen=True)
class DistributedFeatureSet:
    allow_experimental_conv_tp: bool = False
    allow_experimental_spikformer_tp: bool = False
    allow_zero_optimizer: bool = True


@dataclass(frozen=True)
class SNNDistributedPlan:
    """The decision of ``plan()``.  ``tensor_parallel_plan`` (module path -> style) is frozen on
    construction; its keys must be candidates found by the analysis."""
    mode: str
    objective: str
    topology: SNNDistributedTopology
    model_family: str
    backend: str
    batch_size: int
    optimizer_strategy: str
    memopt_level: int
    rationale: Tuple[str, ...]
    notes: Tuple[str, ...]
    tensor_parallel_roots: Optional[Tuple[str, ...]] = None
    tensor_parallel_plan: Optional[Mapping[str, TensorParallelStyle]] = None
    experimental_features: DistributedFeatureSet = DistributedFeatureSet()

    def __post_init__(self):
        if self.tensor_parallel_plan is not None:
            object.__setattr__(self, "tensor_parallel_plan", MappingProxyType(dict(self.tensor_parallel_plan)))

    @property
    def mesh_shape(self) -> Tuple[int, ...]:
        return self.topology.mesh_shape

    @property
    def tp_mesh_dim(self) -> int:
        names = self.topology.ordered_dim_names
        return names.index("tp") if "tp" in names else 0

    @property
    def dp_mesh_dim(self) -> Optional[int]:
        names = self.topology.ordered_dim_names
        return names.index("dp") if "dp" in names else None


@dataclass(frozen=True)
class SNNDistributedRecommendation:
    prefer: str
    model: str
    world_size: int
    mode: str
    optimizer_sharding: str = "none"
    memopt_level: int = 0
    mesh_shape: Optional[Tuple[int, ...]] = None
    tp_mesh_dim: int = 0
    dp_mesh_dim: Optional[int] = None
    pp_microbatches: Optional[int] = None
    pp_memopt_stage_budget_ratio: float = 0.5
    pp_schedule: str = "1f1b"
    pp_virtual_stages: int = 1
    pp_layout: Optional[Tuple[int, ...]] = None
    pp_delay_wgrad: bool = False
    rationale: Tuple[str, ...] = ()


def recommended_pipeline_microbatches(batch_size: int, num_stages: int) -> int:
    """Largest divisor of ``batch_size`` in ``[num_stages, min(batch_size, 4 * num_stages)]``."""
    if batch_size <= 0:
        raise ValueError(f"batch_size must be positive, but got {batch_size}.")
    if num_stages <= 0:
        raise ValueError(f"num_stages must be positive, but got {num_stages}.")
    if batch_size < num_stages:
        raise ValueError(f"batch_size ({batch_size}) must be >= num_stages ({num_stages}) for pipeline parallelism with the "
                         "current microbatch splitting implementation.")
    target = min(batch_size, num_stages * 4)
    for candidate in range(target, num_stages - 1, -1):
        if batch_size % candidate == 0:
            return candidate
    raise ValueError(f"batch_size ({batch_size}) must be divisible by at least one microbatch count in [{num_stages}, {target}] "
                     "for pipeline parallelism.")


def _two_d_mesh(world_size: int) -> Optional[Tuple[int, int]]:
    return None if world_size < 4 or world_size % 2 else (world_size // 2, 2)


def recommend_snn_distributed_strategy(model: str, world_size: int, prefer: str, batch_size: int, backend: str = "inductor",
                                       zero_redundancy_optimizer_available: Optional[bool] = None,
                                       pipelining_available: Optional[bool] = None, fsdp2_available: Optional[bool] = None,
                                       tensor_parallel_available: Optional[bool] = None) -> SNNDistributedRecommendation:
    """speed -> data parallel (+ZeRO) (FSDP2 x TP for the CIFAR10-DVS VGG); memory -> FSDP2 x TP, TP,
    FSDP2 or DP with memopt level 1; capacity -> pipeline parallel when the batch allows it, else the
    memory strategy.  One rank -> no parallelism."""
    prefer = prefer.lower()
    if prefer not in SNN_DISTRIBUTED_PREFERENCES:
        raise ValueError(f"Unsupported prefer='{prefer}'. Expected one of {SNN_DISTRIBUTED_PREFERENCES}.")
    zero = ZERO_REDUNDANCY_OPTIMIZER_AVAILABLE if zero_redundancy_optimizer_available is None else zero_redundancy_optimizer_available
    pipe = PIPELINING_AVAILABLE if pipelining_available is None else pipelining_available
    fsdp = FSDP2_AVAILABLE if fsdp2_available is None else fsdp2_available
    tp = TENSOR_PARALLEL_AVAILABLE if tensor_parallel_available is None else tensor_parallel_available
    family = "spikformer" if model.startswith("spikformer") else model
    why: List[str] = [f"prefer='{prefer}' with model='{family}', world_size={world_size}, backend='{backend}'."]

    def result(mode: str, **kw) -> SNNDistributedRecommendation:
        return SNNDistributedRecommendation(prefer=prefer, model=model, world_size=world_size, mode=mode, rationale=tuple(why), **kw)

    if world_size <= 1:
        why.append("Single-rank run keeps the simplest local path with no distributed overhead." if prefer == "speed"
                   else "Single-rank run falls back to local training and uses memopt for memory savings.")
        return result("none", memopt_level=0 if prefer == "speed" else 1)

    if prefer == "speed":
        mesh = _two_d_mesh(world_size)
        if family == "cifar10dvs_vgg" and fsdp and tp and mesh is not None:
            why.append("Use fsdp2_tp on multi-GPU CIFAR10DVSVGG because benchmarks show the best global throughput there.")
            return result("fsdp2_tp", mesh_shape=mesh, tp_mesh_dim=1, dp_mesh_dim=0)
        why.append("Use data parallel training for the simplest throughput-oriented path, enabling ZeRO optimizer state "
                   "sharding when available.")
        return result("dp", optimizer_sharding="zero" if zero else "none", dp_mesh_dim=0)

    if prefer == "memory":
        mesh = _two_d_mesh(world_size)
        if fsdp and tp and mesh is not None:
            why.append("Combine FSDP2 and TP to shard both parameters and activations, and enable memopt level 1 for the "
                       "strongest memory reduction.")
            return result("fsdp2_tp", memopt_level=1, mesh_shape=mesh, tp_mesh_dim=1, dp_mesh_dim=0)
        if tp:
            why.append("Use tensor parallel with memopt level 1 when two-dimensional FSDP2+TP is unavailable.")
            return result("tp", memopt_level=1, mesh_shape=(world_size,))
        if fsdp:
            why.append("Fall back to FSDP2 with memopt level 1 when TP is unavailable.")
            return result("fsdp2", memopt_level=1, dp_mesh_dim=0)
        why.append("Fall back to DP + memopt level 1 because TP/FSDP2 are unavailable.")
        return result("dp", optimizer_sharding="zero" if zero else "none", memopt_level=1, dp_mesh_dim=0)

    # capacity
    if pipe:
        virtual = 2 if (batch_size >= world_size * 2 and world_size >= 2) else (1 if batch_size >= world_size else 0)
        if virtual == 0:
            why.append("Pipeline parallelism is skipped because the global batch is smaller than the number of physical stages.")
        else:
            why.append("Use pipeline parallelism with memopt level 1 when capacity is the priority; prefer the interleaved "
                       "schedule when several virtual stages per rank are possible.")
            return result("pp", memopt_level=1, pp_microbatches=recommended_pipeline_microbatches(batch_size, world_size * virtual),
                          pp_memopt_stage_budget_ratio=0.5, pp_schedule="interleaved" if virtual > 1 else "1f1b",
                          pp_virtual_stages=virtual)
        why.append("Pipeline parallelism is infeasible for this batch size, so capacity preference falls back to the strongest "
                   "memory-oriented strategy.")
    else:
        why.append("Pipeline APIs are unavailable, so capacity preference falls back to the strongest memory-oriented strategy.")
    fb = recommend_snn_distributed_strategy(model, world_size, "memory", batch_size, backend, zero, False, fsdp, tp)
    return replace(fb, prefer=prefer, rationale=tuple(why + list(fb.rationale[1:])))
