"""Strategy recommendation and the frozen execution plan of Analyze -> Plan -> Apply.

Public names follow ``spikingjelly/activation_based/distributed/planner.py:60-110,257-490``.  The recommender is a rule
table: for each preference an ordered list of ``(applies?, build)`` pairs evaluated against one :class:`_Situation`; the
first rule that applies wins, and every rule records why it was taken or passed over."""
from __future__ import annotations

import importlib
from dataclasses import dataclass, field, replace
from types import MappingProxyType
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple, Union

from . import _schema
from .topology import SNNDistributedTopology

__all__ = ["SNN_DISTRIBUTED_PREFERENCES", "DistributedFeatureSet", "SNNDistributedPlan", "SNNDistributedRecommendation",
           "TensorParallelStyle", "recommended_pipeline_microbatches", "recommend_snn_distributed_strategy",
           "FSDP2_AVAILABLE", "ZERO_REDUNDANCY_OPTIMIZER_AVAILABLE", "PIPELINING_AVAILABLE", "TENSOR_PARALLEL_AVAILABLE"]

TensorParallelStyle = Union[str, Any]
SNN_DISTRIBUTED_PREFERENCES = ("speed", "memory", "capacity")


def _importable(module: str, attribute: str) -> bool:
    try:
        return hasattr(importlib.import_module(module), attribute)
    except ImportError:
        return False


FSDP2_AVAILABLE = _importable("torch.distributed.fsdp", "fully_shard")
ZERO_REDUNDANCY_OPTIMIZER_AVAILABLE = _importable("torch.distributed.optim", "ZeroRedundancyOptimizer")
PIPELINING_AVAILABLE = _importable("torch.distributed.pipelining", "PipelineStage")
#: tensor parallelism here runs on plain process groups and needs nothing optional
TENSOR_PARALLEL_AVAILABLE = True


@dataclass(frozen=True)
class DistributedFeatureSet:
    """Opt-ins that ``plan()`` / ``apply()`` honour."""
    allow_experimental_conv_tp: bool = False
    allow_experimental_spikformer_tp: bool = False
    allow_zero_optimizer: bool = True


@dataclass(frozen=True)
class SNNDistributedPlan:
    """What ``plan()`` decided.  ``tensor_parallel_plan`` (module path -> style) becomes read-only on construction."""
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
        at = self.topology.axis("tp")
        return 0 if at is None else at

    @property
    def dp_mesh_dim(self) -> Optional[int]:
        return self.topology.axis("dp")


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
    """The largest micro-batch count between ``num_stages`` and ``4 * num_stages`` (at most ``batch_size``) that divides
    the batch: enough micro-batches to fill the pipeline, equal sizes so that no stage sees a ragged one."""
    batch = _schema.positive(batch_size, "batch_size")
    stages = _schema.positive(num_stages, "num_stages")
    if batch < stages:
        raise ValueError(f"batch_size: {batch} samples cannot feed {stages} pipeline stages (one micro-batch per stage is the minimum)")
    ceiling = min(batch, 4 * stages)
    fitting = [m for m in range(stages, ceiling + 1) if batch % m == 0]
    if not fitting:
        raise ValueError(f"batch_size: {batch} has no divisor between {stages} and {ceiling}, so it cannot be cut into equal micro-batches")
    return fitting[-1]


# ----------------------------------------------------------------------------------------------- rule table
@dataclass
class _Situation:
    family: str
    model: str
    world: int
    batch: int
    backend: str
    zero: bool
    pipe: bool
    fsdp: bool
    tp: bool
    why: List[str] = field(default_factory=list)

    @property
    def grid(self) -> Optional[Tuple[int, int]]:
        """(replicas, 2) when the ranks split into a two-axis mesh, else None."""
        return (self.world // 2, 2) if self.world >= 4 and self.world % 2 == 0 else None

    @property
    def zero_or_none(self) -> str:
        return "zero" if self.zero else "none"

    def virtual_stages(self) -> int:
        """Pipeline stages per rank the batch can feed: 2 (interleaved), 1, or 0 (no pipeline possible)."""
        if self.batch >= 2 * self.world:
            return 2
        return 1 if self.batch >= self.world else 0


_Fields = Dict[str, Any]
_Rule = Tuple[Callable[[_Situation], bool], Callable[[_Situation], _Fields], str]


def _hybrid(memopt: int) -> Callable[[_Situation], _Fields]:
    return lambda s: dict(mode="fsdp2_tp", memopt_level=memopt, mesh_shape=s.grid, tp_mesh_dim=1, dp_mesh_dim=0)


def _pipeline(s: _Situation) -> _Fields:
    v = s.virtual_stages()
    return dict(mode="pp", memopt_level=1, pp_virtual_stages=v, pp_schedule="interleaved" if v > 1 else "1f1b",
                pp_microbatches=recommended_pipeline_microbatches(s.batch, s.world * v), pp_memopt_stage_budget_ratio=0.5)


_MEMORY_RULES: Sequence[_Rule] = (
    (lambda s: s.fsdp and s.tp and s.grid is not None, _hybrid(1),
     "parameters sharded over one mesh axis (FSDP2) and activations over the other (tensor parallel), plus input-compressed "
     "checkpointing (memopt level 1): the largest saving available"),
    (lambda s: s.tp, lambda s: dict(mode="tp", memopt_level=1, mesh_shape=(s.world,)),
     "no two-axis mesh possible here, so tensor parallelism alone with memopt level 1"),
    (lambda s: s.fsdp, lambda s: dict(mode="fsdp2", memopt_level=1, dp_mesh_dim=0),
     "tensor parallelism unavailable: FSDP2 with memopt level 1"),
    (lambda s: True, lambda s: dict(mode="dp", memopt_level=1, dp_mesh_dim=0, optimizer_sharding=s.zero_or_none),
     "neither tensor parallelism nor FSDP2 available: data parallel with memopt level 1"),
)

_RULES: Dict[str, Sequence[_Rule]] = {
    "speed": (
        (lambda s: s.family == "cifar10dvs_vgg" and s.fsdp and s.tp and s.grid is not None, _hybrid(0),
         "the CIFAR10-DVS VGG measured fastest as FSDP2 x tensor parallel on several GPUs"),
        (lambda s: True, lambda s: dict(mode="dp", dp_mesh_dim=0, optimizer_sharding=s.zero_or_none),
         "data parallel is the shortest path to throughput; optimizer state is sharded (ZeRO-1) where torch offers it"),
    ),
    "memory": _MEMORY_RULES,
    "capacity": (
        (lambda s: s.pipe and s.virtual_stages() > 0, _pipeline,
         "pipeline parallel with memopt level 1 fits the largest model; two virtual stages per rank (interleaved) when the batch "
         "can feed them"),
    ) + tuple(_MEMORY_RULES),
}

_PASSED_OVER = {
    "capacity": lambda s: ("pipeline parallelism is not available in this PyTorch build" if not s.pipe else
                           f"a batch of {s.batch} cannot feed {s.world} pipeline stages") + "; falling back to the memory rules",
}


def recommend_snn_distributed_strategy(model: str, world_size: int, prefer: str, batch_size: int, backend: str = "inductor",
                                       zero_redundancy_optimizer_available: Optional[bool] = None,
                                       pipelining_available: Optional[bool] = None, fsdp2_available: Optional[bool] = None,
                                       tensor_parallel_available: Optional[bool] = None) -> SNNDistributedRecommendation:
    """``speed``: data parallel (+ ZeRO-1), or FSDP2 x TP for the CIFAR10-DVS VGG.  ``memory``: FSDP2 x TP, else TP, else
    FSDP2, else DP — each with memopt level 1.  ``capacity``: pipeline parallel if the batch can feed the stages, else the
    memory rules.  A single rank always trains locally.  The ``*_available`` arguments override what was detected at import."""
    prefer = _schema.one_of(prefer, SNN_DISTRIBUTED_PREFERENCES, "prefer")

    def given(value: Optional[bool], detected: bool) -> bool:
        return detected if value is None else bool(value)

    s = _Situation(family="spikformer" if model.startswith("spikformer") else model, model=model, world=int(world_size),
                   batch=int(batch_size), backend=backend, zero=given(zero_redundancy_optimizer_available, ZERO_REDUNDANCY_OPTIMIZER_AVAILABLE),
                   pipe=given(pipelining_available, PIPELINING_AVAILABLE), fsdp=given(fsdp2_available, FSDP2_AVAILABLE),
                   tp=given(tensor_parallel_available, TENSOR_PARALLEL_AVAILABLE))
    s.why.append(f"asked for {prefer!r}: model family {s.family!r}, {s.world} rank(s), batch {s.batch}, backend {backend!r}")
    if s.world <= 1:
        local_memopt = 0 if prefer == "speed" else 1
        s.why.append("one rank: local training" + ("" if local_memopt == 0 else " with memopt level 1 for the memory saving"))
        fields: _Fields = dict(mode="none", memopt_level=local_memopt)
    else:
        rules = _RULES[prefer]
        chosen = next(i for i, (applies, _, _) in enumerate(rules) if applies(s))
        if chosen > 0 and prefer in _PASSED_OVER:
            s.why.append(_PASSED_OVER[prefer](s))
        _, build, reason = rules[chosen]
        s.why.append(reason)
        fields = build(s)
    return SNNDistributedRecommendation(prefer=prefer, model=model, world_size=s.world, rationale=tuple(s.why), **fields)
